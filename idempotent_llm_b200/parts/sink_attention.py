"""Causal grouped-query attention with short filters, a partial rotation, a sink and an output gate (a mixer).

In this file's notation, for the mixer's input h of one sequence (positions t = 0 .. T-1):

    q, k, v = Wq h, Wk h, Wv h                      no bias; q, k heads of ``key_dim``, v heads of ``value_dim``
    q, k, v <- filter(q), filter(k), filter(v)      per channel, ``conv_taps`` taps, causal, zeros before t = 0
    q, k    <- turn(q), turn(k)                     the first ``position.dim`` dims of each head, by position
    s_tj    = scale * q_t . k_j  (j <= t)           q-head i reads kv-head i // (heads / kv_heads)
    a_tj    = exp(s_tj) / (sum_j' exp(s_tj') + exp(sink_i))
    o_t     = (sum_j a_tj v_j) * sigmoid(Wg h_t)    heads merged as channel = head * value_dim + d
    out     = Wo o

Scores, softmax and the filters run in 32-bit.  k and v are written once into the paged cache after filter and
rotation; a filter's last ``conv_taps - 1`` inputs (the projections' outputs) are per-sequence state.

The mixer can run alone (``forward``) or as a branch of a parallel mixer, which makes one matrix product of
all branches' input projections and one of their outputs: ``in_weight`` / ``out_weight`` / ``inner`` / ``mix``.
"""

from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..weights.loader import TensorDecl
from .base import MIXERS, POSITIONS, Mixer


@MIXERS.register("sink_attention")
class SinkAttention(Mixer):
    @staticmethod
    def _channels(s):
        """Filtered channels: q, k, v."""
        return (s.n_heads + s.n_kv_heads) * s.key_dim + s.n_kv_heads * s.value_dim

    @classmethod
    def declare(cls, spec, prefix):
        s, nm = spec, spec.names
        rows = {nm.q: s.n_heads * s.key_dim, nm.k: s.n_kv_heads * s.key_dim, nm.v: s.n_kv_heads * s.value_dim}
        d = [TensorDecl(prefix + n, (r, s.hidden)) for n, r in rows.items()]
        if s.conv_taps > 1:
            d += [TensorDecl(prefix + n + nm.conv, (r, s.conv_taps), init="filter") for n, r in rows.items()]
        if s.sink:
            d.append(TensorDecl(prefix + nm.sink, (s.n_heads,), init="unit_normal"))
        if s.gate:
            d.append(TensorDecl(prefix + nm.gate, (s.n_heads * s.value_dim, s.hidden)))
        d.append(TensorDecl(prefix + nm.o, (s.hidden, s.n_heads * s.value_dim)))
        return d

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        s = spec
        return CacheNeed(kind="full", n_kv_heads=s.n_kv_heads, head_dim=s.key_dim,
                         k_row=(s.n_kv_heads, s.key_dim), v_row=(s.n_kv_heads, s.value_dim),
                         state_shape=((s.conv_taps - 1) * cls._channels(s),) if s.conv_taps > 1 else None)

    def __init__(self, spec, weights, prefix, rt):
        s, nm = spec, spec.names
        if s.n_heads % s.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.spec, self.rt = spec, rt
        mats = [weights[prefix + n] for n in (nm.q, nm.k, nm.v)] + ([weights[prefix + nm.gate]] if s.gate else [])
        self.in_weight = torch.cat([m.to(rt.dtype) for m in mats], dim=0).contiguous()
        self.out_weight = weights[prefix + nm.o].to(rt.dtype).contiguous()
        self.inner = s.n_heads * s.value_dim
        self.channels = self._channels(s)
        if s.conv_taps > 1:
            self.w_conv = torch.cat([weights[prefix + n + nm.conv].to(torch.float32) for n in (nm.q, nm.k, nm.v)],
                                    dim=0).contiguous()
        else:
            self.w_conv = torch.ones((self.channels, 1), dtype=torch.float32, device=rt.device)
        self.sink = weights[prefix + nm.sink].to(torch.float32).contiguous() if s.sink else None
        self.position = None
        if s.position is not None:
            variant = getattr(s.position, "variant", None)
            if variant not in ("half_partial", "half_whole_head") or s.position.dim > s.key_dim or s.position.dim % 2:
                raise ValueError(f"sink attention: position encoding variant {variant!r} over {s.position.dim} of "
                                 f"{s.key_dim} dims is not built; the kernels turn dim i with dim i + dim / 2 over the "
                                 f"first `dim` dims of a head ('half_partial')")
            self.position = POSITIONS.get(s.position.kind)(s.position, weights, prefix, rt)

    # -- as a branch: columns [col0, col0 + in_weight rows) of `proj` are this mixer's projections of the step
    def mix(self, proj, col0, ctx, kv, state, out, out_col, out_scale):
        s, K = self.spec, self.rt.kernels
        cs = self.position.tables(ctx) if self.position is not None else None
        q = K.conv_qkv_cache(proj, col0, self.w_conv, state, s.n_heads, s.n_kv_heads, s.key_dim, s.value_dim, cs, kv, ctx)
        if s.conv_taps > 1 and not ctx.single_token:
            K.conv_state_update(proj, col0, self.channels, s.conv_taps, state, ctx)
        gate = proj[:, col0 + self.channels:col0 + self.channels + self.inner] if s.gate else None
        if K.attention_tc_fits(kv, s.key_dim, s.value_dim):
            # on the tensor cores, for prompts and single tokens alike; gate and constant in a pass of their own
            o = K.attention_tc(q, kv, ctx, s.softmax_scale, sink=self.sink)
            K.gate_scale(o, gate, proj.shape[1], out_scale, out, out_col)
        else:
            K.attention_sink(q, kv, ctx, s.softmax_scale, self.sink, gate, proj.shape[1], out, out_col, out_scale)

    def forward(self, x, ctx, kv, state, writes_cache: bool):
        if not writes_cache:
            raise ValueError("this mixer writes its own keys and values")
        K = self.rt.kernels
        proj = K.gemm_store(x, self.in_weight, pad=True)
        out = torch.empty((x.shape[0], self.inner), dtype=self.rt.dtype, device=x.device)
        self.mix(proj, 0, ctx, kv, state, out, 0, 1.0)
        return K.gemm(out, self.out_weight, pad=True)
