"""Causal attention whose keys and values come from one latent vector per token (a mixer).

In this file's notation, for the mixer's input h of one sequence (positions t = 0 .. T-1) and head i:

    [qn_i | qr_i]_t = rows of Wq h_t                  ``plain_dim`` unrotated and ``rot_dim`` rotated dims per head
    [a_t | b_t]     = Wd h_t                          ``kv_rank`` and ``rot_dim`` numbers
    c_t             = a_t / sqrt(mean(a_t^2) + eps) * g
    r_t             = turn(b_t, t),  qr <- turn(qr, t)        neighbours (2j, 2j+1) by angle t f_j, times a magnitude
    s_tj            = scale * (qn_i . Uk_i c_j + qr_i . r_j)   (j <= t)
    w_tj            = exp(s_tj) / (sum_j' exp(s_tj') [+ exp(sink_i)])
    out_t           = Wo [.. | Uv_i sum_j w_tj c_j | ..]

A token keeps the row ``[c_t | r_t]`` and nothing per head.  The kernels work in the latent's space: the query
becomes ``[Uk_i^T qn_i | qr_i]``, every head scores the same cached rows, the context is a weighted sum of ``c``, and
``Uv_i`` is applied once to that sum: the same sums in another order.  Scores, softmax, the latent's norm and the
rotation are 32-bit; matrices, the cached rows and the products' inputs are in the storage dtype.

A step of whole prompts (every sequence from its first token) has many queries per cached row; in bfloat16, with
heads that fit the tensor-core attention kernel, it makes every head's keys and values from the step's rows with one
matrix product and runs that kernel over pages of the step's own (``_whole_prompts``).  The cache receives the same
rows either way, so later single tokens read what the prompt left.
"""

from __future__ import annotations

import torch

from ..cache.sequence_cache import KVView
from ..cache.spec import CacheNeed
from ..weights.loader import TensorDecl
from .base import MIXERS, POSITIONS, Mixer


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    accepts_residual = True
    same_bits_across_steps = False      # whole prompts, portions and single tokens take different kernels

    @classmethod
    def declare(cls, spec, prefix):
        s, nm = spec, spec.names
        d = [TensorDecl(prefix + nm.q, (s.n_heads * (s.plain_dim + s.rot_dim), s.hidden)),
             TensorDecl(prefix + nm.down, (s.kv_rank + s.rot_dim, s.hidden)),
             TensorDecl(prefix + nm.down_norm, (s.kv_rank,), init="one_plus_normal"),
             TensorDecl(prefix + nm.up_k, (s.n_heads * s.plain_dim, s.kv_rank)),
             TensorDecl(prefix + nm.up_v, (s.n_heads * s.value_dim, s.kv_rank))]
        if s.sink:
            d.append(TensorDecl(prefix + nm.sink, (s.n_heads,), init="unit_normal"))
        d.append(TensorDecl(prefix + nm.o, (s.hidden, s.n_heads * s.value_dim)))
        return d

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        # one row per token for all heads: the latent and the shared rotated key part side by side; no value rows
        row = spec.kv_rank + spec.rot_dim
        return CacheNeed(kind="full", n_kv_heads=1, head_dim=row, k_row=(1, row), v_row=(1, 0))

    def __init__(self, spec, weights, prefix, rt):
        s, nm = spec, spec.names
        self.spec, self.rt = spec, rt
        if s.kv_rank > rt.kernels.latent_max_rank():
            raise ValueError(f"latent attention: a latent of {s.kv_rank} numbers is more than the kernels hold "
                             f"({rt.kernels.latent_max_rank()})")
        self.rot_dims, self.position, self.magnitude = 0, None, 1.0
        if s.position is not None:
            variant = getattr(s.position, "variant", None)
            if variant != "interleaved" or s.position.dim > s.rot_dim or s.position.dim % 2:
                raise ValueError(f"latent attention: position encoding variant {variant!r} over {s.position.dim} of "
                                 f"{s.rot_dim} dims is not built; the kernels turn neighbours (2j, 2j+1) of the rotated part "
                                 f"('interleaved')")
            self.position = POSITIONS.get(s.position.kind)(s.position, weights, prefix, rt)
            self.rot_dims = s.position.dim
            self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        H, dn, dv, R = s.n_heads, s.plain_dim, s.value_dim, s.kv_rank
        # q and the down projection are one product (rows one after another)
        self.w_in = torch.cat([weights[prefix + nm.q].to(rt.dtype), weights[prefix + nm.down].to(rt.dtype)], dim=0).contiguous()
        self.q_cols = H * (dn + s.rot_dim)
        self.down_norm = weights[prefix + nm.down_norm].to(torch.float32).contiguous()
        # per head [in, out] with `out` contiguous: Uk_i as stored (plain_dim x rank), Uv_i transposed (rank x value_dim)
        self.uk = weights[prefix + nm.up_k].to(rt.dtype).reshape(H, dn, R).contiguous()
        self.uv_t = weights[prefix + nm.up_v].to(rt.dtype).reshape(H, dv, R).transpose(1, 2).contiguous()
        self.sink = weights[prefix + nm.sink].to(torch.float32).contiguous() if s.sink else None
        self.w_o = weights[prefix + nm.o].to(rt.dtype).contiguous()
        self.pad = {"pad": True} if rt.dtype == torch.bfloat16 and (s.hidden % 8 or (H * dv) % 8) else {}
        # whole prompts on the tensor cores: heads padded to a head size that kernel has
        self.tc_hd = 0
        K = rt.kernels
        if (rt.dtype == torch.bfloat16 and getattr(K, "fused", False) and getattr(K, "attention_impl", "") == "tcgen05"
                and not self.pad and (R + s.rot_dim) % 8 == 0):
            need = max(dn + s.rot_dim, dv)
            self.tc_hd = 64 if need <= 64 else 128 if need <= 128 else 0
        if self.tc_hd:
            hd = self.tc_hd
            up = torch.zeros((H * dn + H * dv, R + s.rot_dim), dtype=rt.dtype, device=rt.device)
            up[:H * dn, :R] = weights[prefix + nm.up_k].to(rt.dtype)
            up[H * dn:, :R] = weights[prefix + nm.up_v].to(rt.dtype)
            self.w_up = up.contiguous()                      # [Uk ; Uv] over a cached row (zero over its rotated part)
            wo = torch.zeros((s.hidden, H, hd), dtype=rt.dtype, device=rt.device)
            wo[:, :, :dv] = self.w_o.view(s.hidden, H, dv)
            self.w_o_padded = wo.view(s.hidden, H * hd).contiguous()

    # steps of whole prompts take the per-head kernel from this many tokens in the longest prompt on
    WHOLE_FROM = 32

    def _step_pages(self, ctx):
        """A block table of the step's own: sequence i's pages one after another (made once a step)."""
        made = ctx.memo.get("latent_step_pages")
        if made is None:
            page = self.rt.kernels.page
            table = torch.zeros((max(ctx.host_slots) + 1, max(-(-n // page) for n in ctx.host_q_lens)), dtype=torch.int32)
            at = 0
            for slot, n in zip(ctx.host_slots, ctx.host_q_lens):
                pages = -(-n // page)
                table[slot, :pages] = torch.arange(at, at + pages, dtype=torch.int32)
                at += pages
            made = ctx.memo["latent_step_pages"] = (table.to(self.rt.device), at)
        return made

    def _whole_prompts(self, proj, cs, ctx, kv, residual):
        s, K, hd = self.spec, self.rt.kernels, self.tc_hd
        rows = K.latent_kv_finish(proj, self.q_cols, s.kv_rank, s.rot_dim, self.rot_dims, self.down_norm, s.eps, cs,
                                  self.magnitude, kv, ctx, keep_rows=True)
        up = K.gemm_store(rows, self.w_up)                                  # 32-bit [N, H * plain_dim + H * value_dim]
        table, n_pages = self._step_pages(ctx)
        q, k, v = K.latent_expand_pack(proj, up, rows, s.n_heads, s.plain_dim, s.rot_dim, s.value_dim, s.kv_rank,
                                       self.rot_dims, cs, self.magnitude, hd, table, n_pages, ctx)
        own = KVView(k=k, v=v, table=table, ring=0, n_kv_heads=s.n_heads, head_dim=hd, window=None)
        o = K.attention_tc(q, own, ctx, s.softmax_scale, sink=self.sink)    # [N, H * hd]
        if residual is not None:
            K.gemm_residual(o, self.w_o_padded, residual)
            return None
        return K.gemm(o, self.w_o_padded)

    def forward(self, x, ctx, kv, state, writes_cache: bool, residual=None):
        """Returns the delta ``[1, N, hidden]``, or None after adding it into ``residual`` in place."""
        if not writes_cache:
            raise ValueError("this mixer writes its own cache entry")
        s, K = self.spec, self.rt.kernels
        cs = self.position.tables(ctx) if self.position is not None else None
        proj = K.gemm_store(x, self.w_in, **self.pad)                       # 32-bit [N, q columns + rank + rot_dim]
        if self.tc_hd and not ctx.single_token and ctx.max_q_len >= self.WHOLE_FROM and not any(ctx.host_starts):
            return self._whole_prompts(proj, cs, ctx, kv, residual)
        K.latent_kv_finish(proj, self.q_cols, s.kv_rank, s.rot_dim, self.rot_dims, self.down_norm, s.eps, cs,
                           self.magnitude, kv, ctx)
        # queries into the latent's space, their rotated part turned: [N, H, rank + rot_dim], 32-bit
        qa = K.headwise(proj, 0, s.n_heads, s.plain_dim + s.rot_dim, self.uk, tail=s.rot_dim, rot_dims=self.rot_dims,
                        cs=cs, mag=self.magnitude, out_f32=True)
        c = K.latent_attention(qa, kv, ctx, s.kv_rank, s.softmax_scale, sink=self.sink)     # 32-bit [N, H * rank]
        o = K.headwise(c, 0, s.n_heads, s.kv_rank, self.uv_t).view(x.shape[0], s.n_heads * s.value_dim)
        if residual is not None and getattr(K, "fused", False) and not self.pad:
            K.gemm_residual(o, self.w_o, residual)
            return None
        return K.gemm(o, self.w_o, **self.pad)
