"""A layer that norms every sublayer's input and output, and the per-layer token input that may end it.

    h += post_m(mixer(pre_m(h)))
    h += post_f(ff(pre_f(h)))              if the layer has a feed-forward
    h += R(P (act(S h) * e[token]))        if the layer has a token side input (``TokenSide``)

The stream stays 32-bit.  The norm behind a sublayer and the norm (or plain cast) in front of the next one
are one kernel over the row (``post_pre_norm``), which is why the four norms must be plain RMS norms.
"""

from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, NormedDelta, Part
from .mlp import ACTIVATIONS


class TokenSide(Part):
    """``y = P (act(S x) * e)`` with ``e`` this layer's columns of the token's row of a table that all layers
    share; the caller norms ``y`` and adds it."""

    @classmethod
    def declare(cls, spec, prefix):
        s = spec
        return [TensorDecl(s.table, (s.vocab_size, s.table_width)),       # shared: declared by every layer alike
                TensorDecl(prefix + s.gate, (s.dim, s.hidden)),
                TensorDecl(prefix + s.proj, (s.hidden, s.dim)),
                TensorDecl(prefix + s.norm, (s.hidden,), init="one_plus_normal")]

    def __init__(self, spec, weights, prefix, rt):
        s = spec
        if s.activation not in ACTIVATIONS:
            raise ValueError(f"activation {s.activation!r} is not built; known: {sorted(ACTIVATIONS)}")
        self.spec, self.rt = spec, rt
        self.act = ACTIVATIONS[s.activation]
        self.table = rt.shared_tensor(weights, s.table, rt.dtype)
        self.w_gate = weights[prefix + s.gate].to(rt.dtype).contiguous()
        self.w_proj = weights[prefix + s.proj].to(rt.dtype).contiguous()
        self.norm = weights[prefix + s.norm].to(torch.float32).contiguous()

    def forward(self, x, ctx):
        """x: the stream in the storage dtype ``[N, hidden]``; returns 32-bit ``[N, hidden]``, not yet normed."""
        K, s = self.rt.kernels, self.spec
        g = K.token_gate(K.gemm_store(x, self.w_gate, pad=True), ctx.tokens, self.table, s.col0, self.act)
        return K.gemm_store(g, self.w_proj, pad=True)


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    @staticmethod
    def _norms(spec):
        named = [("mixer_norm", spec.mixer_norm), ("mixer_post_norm", spec.mixer_post_norm)]
        if spec.feed_forward is not None:
            named += [("feed_forward_norm", spec.feed_forward_norm), ("feed_forward_post_norm", spec.feed_forward_post_norm)]
        for name, n in named:
            if n is None or n.kind != "rmsnorm":
                raise ValueError(f"a sandwich layer's {name} must be an RMS norm (its kernels norm and add in one pass)")
        return named

    @classmethod
    def declare(cls, spec, prefix=None):
        p = spec.prefix
        d = []
        for _, n in cls._norms(spec):
            d += NORMS.get(n.kind).declare(n, p)
        d += MIXERS.get(spec.mixer.kind).declare(spec.mixer, p)
        if spec.feed_forward is not None:
            d += FEED_FORWARDS.get(spec.feed_forward.kind).declare(spec.feed_forward, p)
        if spec.token_side is not None:
            d += TokenSide.declare(spec.token_side, p)
        return d

    def __init__(self, spec, weights, prefix, rt):
        p = spec.prefix
        self.spec, self.rt = spec, rt
        for name, n in self._norms(spec):
            setattr(self, name, NORMS.get(n.kind)(n, weights, p, rt))
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, weights, p, rt)
        self.feed_forward = self.token_side = None
        if spec.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, weights, p, rt)
        if spec.token_side is not None:
            self.token_side = TokenSide(spec.token_side, weights, p, rt)

    def forward(self, h, pending, ctx, kv, state, writes_cache: bool):
        K = self.rt.kernels
        x = self.mixer_norm.forward(h, pending, ctx)
        y, post = self.mixer.forward(x, ctx, kv, state, writes_cache)[0], self.mixer_post_norm
        if self.feed_forward is not None:
            pre = self.feed_forward_norm
            x = K.post_pre_norm(h, y, post.weight, post.spec.eps, w_pre=pre.weight, eps_pre=pre.spec.eps)
            y, post = self.feed_forward.forward(x, ctx)[0], self.feed_forward_post_norm
        # the norm behind the last sublayer is handed on: the next layer's first norm (or the final one) adds it
        if self.token_side is not None:
            x = K.post_pre_norm(h, y, post.weight, post.spec.eps, cast=True)
            return h, NormedDelta(self.token_side.forward(x, ctx), self.token_side.norm, self.token_side.spec.eps)
        return h, NormedDelta(y, post.weight, post.spec.eps)
