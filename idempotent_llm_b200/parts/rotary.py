"""Rotary position encoding: the step's cos/sin table.

``inv_freq_j = theta ** (-2 j / dim)`` in 64-bit, angle = position * inv_freq in
64-bit, cos and sin rounded to 32-bit (reference: src/detllm/ops/rope.py:25-35
builds its table the same way before quantising it; float form in
src/detllm/prepare.py:137-141).  The table is made once per step and shared by
every layer with the same ``(theta, dim)``; the rotation itself is fused into
the mixer's kernel.
"""

from __future__ import annotations

import math

import torch

from .base import POSITIONS, PositionEncoding


def magnitude(spec) -> float:
    """What cos and sin are multiplied with: ``0.1 ln(factor) + 1`` under a ``RampScaling``, else 1."""
    sc = getattr(spec, "scaling", None)
    return 0.1 * math.log(sc.factor) + 1.0 if sc is not None and hasattr(sc, "fast") else 1.0


def frequencies(spec) -> torch.Tensor:
    """``theta ** (-2 j / dim)`` for ``j < dim / 2`` in 64-bit, then the spec's scaling by wavelength, if any
    (``WavelengthScaling``: short waves kept, long waves divided by the factor, a linear blend between)."""
    j = torch.arange(0, spec.dim // 2, dtype=torch.float64)
    f = float(spec.theta) ** (-2.0 * j / spec.dim)
    sc = getattr(spec, "scaling", None)
    if sc is None:
        return f
    if hasattr(sc, "fast"):                 # RampScaling: slowed down along a ramp over j between two borders
        def at(turns):
            return spec.dim * math.log(sc.original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(spec.theta)))
        lo = max(math.floor(at(sc.fast)), 0)
        hi = min(math.ceil(at(sc.slow)), spec.dim - 1)
        ramp = torch.clamp((j - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / sc.factor * ramp + f * (1.0 - ramp)
    wave = 2.0 * math.pi / f
    s = (sc.original / wave - sc.low) / (sc.high - sc.low)
    blend = (1.0 - s) * f / sc.factor + s * f
    return torch.where(wave < sc.original / sc.high, f, torch.where(wave > sc.original / sc.low, f / sc.factor, blend))


@POSITIONS.register("rotary")
class Rotary(PositionEncoding):
    def __init__(self, spec, weights, prefix, rt):
        if spec.dim % 2:
            raise ValueError(f"rotary dimension {spec.dim} must be even")
        self.spec = spec
        self.rt = rt
        self.inv_freq = frequencies(spec).to(rt.device)
        self.magnitude = magnitude(spec)        # applied by the mixer's kernels (the table holds plain cos and sin)
        sc = getattr(spec, "scaling", None)
        self._key = ("rotary", float(spec.theta), spec.dim, None if sc is None else tuple(sorted(vars(sc).items())))

    def emit(self, prog):
        """The table's two buffers in a step program (made once a step, like ``tables``)."""
        key = self._key
        bufs = prog.shared.get(key)
        if bufs is None:
            per_token = self.spec.dim // 2 * 2 * 4
            bufs = prog.shared[key] = (prog.buffer(f"rotary.{len(prog.shared)}", per_token),
                                       prog.buffer(f"rotary.{len(prog.shared)}.by_dim", per_token))
            prog.rope_table(self.inv_freq, *bufs)
        return bufs

    def tables(self, ctx):
        key = self._key
        t = ctx.memo.get(key)
        if t is None:
            t = self.rt.kernels.rope_table(ctx.positions, self.inv_freq)
            ctx.memo[key] = t
        return t
