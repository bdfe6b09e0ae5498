"""A plain, slow implementation of the Panodra decoder: whole sequences, no cache, one function per mechanism,
64-bit floats on the CPU.  It shares no code with the package: it takes the configuration as the dict config.json
holds and the tensors by name.

The design in this file's notation (T tokens, positions 0 .. T-1, width W):

* stream:   x0 = E[token]
* order:    layers 0 .. start-1 once; then `times` passes over layers start .. stop-1, each pass opened by
            x <- M [x ; x0] (M is [W, 2 W]); then layers stop .. end.  Without a `loop` every layer runs once.
* layer:    x <- x + mixer(D1(x));  x <- x + ff(D2(x))  (the second only with a feed-forward)
* D:        tanh(alpha x) * w + b, element by element (no statistics)
* mixer:    attention through a latent: one vector c_t of `kv_rank` numbers and one rotated key part of `rot_dim`
            numbers per token, from which every head's keys and values are made
* ff:       dense: Wd relu(Wu h)^2;  experts: the token id names `top` experts, the mean of Wd (silu(Wg h) * Wu h)
* output:   logits = cap * tanh(scale * E D_f(x) / cap)
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------- small pieces
def dyt(x: torch.Tensor, alpha, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.tanh(float(alpha) * x) * w + b


def unit_rms(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: dict):
    """(f [dims / 2], magnitude): f_i = base^(-2 i / dims); with `scaling`, waves between two borders are slowed
    down by up to `factor` along a ramp over i, and cos and sin grow by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns):        # the i at which a wave makes `turns` turns over the original length
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, f: torch.Tensor, mag: float) -> torch.Tensor:
    """x [T, ..., dims]: neighbours (2i, 2i+1) turned by positions[t] * f_i."""
    T = x.shape[0]
    a = positions.to(F64)[:, None] * f[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [f.numel()]
    cos, sin = (torch.cos(a) * mag).reshape(shape), (torch.sin(a) * mag).reshape(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * cos - v * sin
    out[..., 1::2] = v * cos + u * sin
    return out


# ------------------------------------------------------------------------------- mixer
def latent_attention(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float,
                     positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h [T, W] -> [T, W].  `m` is the layer's `mixer` dict, `p` the tensors' prefix ('l3.mix.')."""
    T = h.shape[0]
    H, dn, dr, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(T) if positions is None else positions
    f, mag = rotary_frequencies(m["rot"])
    q = (h @ w[p + "q"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_pairs(q[..., dn:], pos, f, mag)
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :R], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, R:], pos, f, mag)                       # one for all heads
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    s = (torch.einsum("thd,jhd->htj", q_plain, k_plain) + torch.einsum("thd,jd->htj", q_rot, k_rot)) * float(m["scale"])
    seen = pos[None, :] <= pos[:, None]
    s = s.masked_fill(~seen[None], -math.inf)
    top = s.max(dim=-1, keepdim=True).values
    sink = w.get(p + "sink")
    if sink is not None:
        top = torch.maximum(top, sink.reshape(H, 1, 1))
    e = torch.exp(s - top)
    z = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        z = z + torch.exp(sink.reshape(H, 1, 1) - top)                   # a score with no key and no value
    a = e / z
    o = torch.einsum("htj,jhd->thd", a, v).reshape(T, H * dv)
    return o @ w[p + "o"].T


# ------------------------------------------------------------------------------- feed-forwards
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def table_experts(h: torch.Tensor, tokens: Sequence[int], mlp: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    top = int(mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t, tok in enumerate(tokens):
        for e in w[p + "table"][tok].tolist()[:top]:
            q = f"{p}e{int(e)}."
            out[t] += (silu(h[t] @ w[q + "gate"].T) * (h[t] @ w[q + "up"].T)) @ w[q + "down"].T / top
    return out


# ------------------------------------------------------------------------------- the model
def layer_order(cfg: dict):
    """[(layer, opens a pass)] in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: Sequence[int], streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  `streams`, if a list, receives x after every layer run."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x0 = w["embed"][torch.tensor(list(tokens))]
    x = x0.clone()
    for i, opens in layer_order(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if opens:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        if L["type"] not in ("latent_attention", "latent_attention_2"):
            raise ValueError(L["type"])
        x = x + latent_attention(dyt(x, w[p + "norm1.alpha"], w[p + "norm1"], w[p + "norm1.b"]), L["mixer"], w,
                                 p + "mix.", eps)
        mlp = L.get("mlp")
        if mlp:
            h = dyt(x, w[p + "norm2.alpha"], w[p + "norm2"], w[p + "norm2.b"])
            x = x + (dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else table_experts(h, tokens, mlp, w, p + "mlp."))
        if streams is not None:
            streams.append(x.clone())
    y = dyt(x, w["final.norm.alpha"], w["final.norm"], w["final.norm.b"]) @ w["embed"].T * float(cfg.get("logit_scale", 1.0))
    cap = cfg.get("logit_softcap")
    return y if not cap else float(cap) * torch.tanh(y / float(cap))
