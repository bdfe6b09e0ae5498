"""Selective state-space mixer with a scalar decay per head (state-space duality form).

In this file's notation, for the mixer's input h_t, with inner = heads * P, N the state size, G groups:

    [z | x | B | C | dt] = W_in h_t                 widths inner, inner, G N, G N, heads
    [x | B | C] <- silu(filter([x | B | C]) + b)    per channel, ``conv_taps`` taps, causal
    dt_t  = softplus(dt_t + dt_bias)                per head
    S_t   = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T        S: [N, P] per head, head i reads group i // (heads / G)
    y_t   = S_t^T C_t + D x_t
    o_t   = norm_parts(y_t * silu(z_t)) * w         ``norm_groups`` equal parts, each by its own root mean square
    out   = W_o o_t

The recurrence, its step sizes and decays, the gate and the norm run in 32-bit.  Per-sequence state: the
filter's last ``conv_taps - 1`` inputs and S, in 32-bit, zero at a sequence's start.

Alone (``forward``) or as a branch of a parallel mixer (``in_weight`` / ``out_weight`` / ``inner`` / ``mix``).
"""

from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..weights.loader import TensorDecl
from .base import MIXERS, Mixer


@MIXERS.register("ssd")
class SSDMixer(Mixer):
    @staticmethod
    def _sizes(s):
        inner, gn = s.heads * s.head_dim, s.groups * s.state
        return inner, gn, inner + 2 * gn            # inner, one of B / C, filtered channels

    @classmethod
    def declare(cls, spec, prefix):
        s, nm = spec, spec.names
        inner, gn, ch = cls._sizes(s)
        d = [TensorDecl(prefix + nm.w_in, (2 * inner + 2 * gn + s.heads, s.hidden))]
        if s.conv_taps > 1:
            d += [TensorDecl(prefix + nm.conv, (ch, s.conv_taps), init="filter"),
                  TensorDecl(prefix + nm.conv_bias, (ch,))]
        d += [TensorDecl(prefix + nm.dt_bias, (s.heads,), init="unit_normal"),
              TensorDecl(prefix + nm.a_log, (s.heads,), init="unit_normal"),
              TensorDecl(prefix + nm.d, (s.heads,), init="one_plus_normal"),
              TensorDecl(prefix + nm.norm, (inner,), init="one_plus_normal"),
              TensorDecl(prefix + nm.o, (s.hidden, inner))]
        return d

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        s = spec
        inner, gn, ch = cls._sizes(s)
        return CacheNeed(kind="none", state_shape=((s.conv_taps - 1) * ch + s.heads * s.state * s.head_dim,))

    def __init__(self, spec, weights, prefix, rt):
        s, nm = spec, spec.names
        if s.heads % s.groups or (s.heads * s.head_dim) % s.norm_groups:
            raise ValueError("heads must be a multiple of groups, and heads * head_dim of norm_groups")
        inner, gn, ch = self._sizes(s)
        self.spec, self.rt = spec, rt
        self.inner, self.gn, self.channels = inner, gn, ch
        self.in_weight = weights[prefix + nm.w_in].to(rt.dtype).contiguous()
        self.out_weight = weights[prefix + nm.o].to(rt.dtype).contiguous()
        f32 = lambda n: weights[prefix + n].to(torch.float32).contiguous()
        if s.conv_taps > 1:
            self.w_conv, self.b_conv = f32(nm.conv), f32(nm.conv_bias)
        else:
            self.w_conv, self.b_conv = torch.ones((ch, 1), dtype=torch.float32, device=rt.device), None
        self.dt_bias, self.a_log, self.d, self.norm = f32(nm.dt_bias), f32(nm.a_log), f32(nm.d), f32(nm.norm)
        self.conv_floats = (s.conv_taps - 1) * ch

    def mix(self, proj, col0, ctx, kv, state, out, out_col, out_scale):
        s, K = self.spec, self.rt.kernels
        conv_state = state[:, :self.conv_floats] if self.conv_floats else None
        xbc = K.short_conv(proj, col0 + self.inner, self.channels, self.w_conv, self.b_conv, 1, conv_state, ctx)
        if s.conv_taps > 1 and not ctx.single_token:
            K.conv_state_update(proj, col0 + self.inner, self.channels, s.conv_taps, conv_state, ctx)
        y = K.ssd_scan(xbc, (0, self.inner, self.inner + self.gn), proj, col0, col0 + 2 * self.inner + 2 * self.gn,
                       self.dt_bias, self.a_log, self.d, state[:, self.conv_floats:], ctx, s.heads, s.groups,
                       s.head_dim, s.state)
        K.ssd_group_norm(y, s.norm_groups, self.norm, s.norm_eps, out_scale, out, out_col)

    def forward(self, x, ctx, kv, state, writes_cache: bool):
        K = self.rt.kernels
        proj = K.gemm_store(x, self.in_weight, pad=True)
        out = torch.empty((x.shape[0], self.inner), dtype=self.rt.dtype, device=x.device)
        self.mix(proj, 0, ctx, None, state, out, 0, 1.0)
        return K.gemm(out, self.out_weight, pad=True)
