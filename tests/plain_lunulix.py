"""A plain, slow implementation of the Lunulix decoder: whole sequences, no cache, no state carried
between calls, one function per mechanism, 64-bit floats on the CPU.  It shares no code with the
package: it takes the configuration as the dict config.json holds and the tensors by name.

The design in this file's notation (T tokens, positions 0 .. T-1):

* stream:   x_0 = E[token] * embedding.scale
* layer:    x <- x + N_1b(mixer(N_1(x)));  x <- x + N_2b(ff(N_2(x)))  (the second only with a feed-forward);
            x <- x + R(P g) with g = gelu(S x) * e_i[token]  (the token's side vector of layer i)
* mixer:    a * attention(h) + b * ssd(h), both reading the same h
* output:   logits = H N_f(x)

N is the RMS norm with a weight, R the same with the side path's weight, gelu the tanh form.
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------- small pieces
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start; the last
    column of w multiplies the current token."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y if bias is None else y + bias


# ------------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2 i / dims), i < dims / 2, then the wavelength-dependent scaling: short waves kept,
    long waves divided by the factor, a linear blend between the two borders."""
    dims = int(rot["dims"])
    i = torch.arange(dims // 2, dtype=F64)
    f = float(rot["base"]) ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = f.clone()
    for n in range(f.numel()):
        wave = 2.0 * math.pi / float(f[n])
        if wave < orig / high:
            continue
        if wave > orig / low:
            out[n] = f[n] / factor
        else:
            s = (orig / wave - low) / (high - low)
            out[n] = (1.0 - s) * f[n] / factor + s * f[n]
    return out


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [T, heads, d]; the first 2 * len(freqs) dims of each head turn, dim i with dim i + len(freqs)."""
    half = freqs.numel()
    ang = positions.to(F64)[:, None] * freqs[None, :]            # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


# ------------------------------------------------------------------------------- left: attention
def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                   sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv]; causal; the softmax's denominator also holds exp(sink_h)."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].reshape(1, 1))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def left_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = int(c["heads"]), int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if c.get("conv"):
        q, k, v = (causal_conv(t, w[p + n + ".conv"]) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    if c.get("rot"):
        f = rotary_frequencies(c["rot"])
        pos = torch.arange(T)
        q, k = rotate(q, pos, f), rotate(k, pos, f)
    o = sink_attention(q, k, v, float(c["scale"]), w.get(p + "sink")).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ------------------------------------------------------------------------------- right: state-space
def ssd_scan(x: torch.Tensor, dt: torch.Tensor, a: torch.Tensor, B: torch.Tensor, C: torch.Tensor,
             D: torch.Tensor) -> torch.Tensor:
    """x [T, heads, P], dt [T, heads], a [heads] (= exp(A_log)), B, C [T, groups, N], D [heads].
    S_t = exp(-a dt_t) S_(t-1) + dt_t B_t x_t^T;  y_t = S_t^T C_t + D x_t, token by token."""
    T, nh, P = x.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(x)
    for h in range(nh):
        g = h // (nh // G)
        S = torch.zeros(N, P, dtype=x.dtype)
        for t in range(T):
            S = torch.exp(-a[h] * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return y


def right_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    nh, P, N, G = int(c["heads"]), int(c["vdim"]), int(c["state"]), int(c["groups"])
    inner = nh * P
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, nh, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = ssd_scan(x, dt, torch.exp(w[p + "A_log"]), B, C, w[p + "D"]).reshape(T, inner)
    y = y * silu(z)
    parts = int(c["norm_groups"])
    y = rms_norm(y.view(T, parts, inner // parts), None, eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, c, eps):
    return (float(c["left_scale"]) * left_mixer(h, w, p + "left.", c["left"])
            + float(c["right_scale"]) * right_mixer(h, w, p + "right.", c["right"], eps))


# ------------------------------------------------------------------------------- the rest of a layer
def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def token_side(x, tokens, w, p, layer: int, dim: int, eps: float):
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w[p + "gate"].T) * e
    return rms_norm(g @ w[p + "proj"].T, w[p + "norm"], eps)


# ------------------------------------------------------------------------------- the model
def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], return_layers: bool = False):
    """Logits [T, vocab] in 64-bit for one whole sequence (and the stream after every layer)."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["embed"][tok] * float(cfg["embedding"]["scale"])
    side = cfg.get("token_side")
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(f"layer type {layer['type']!r}")
        m = parallel_mixer(rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        x = x + rms_norm(m, w[p + "norm1b"], eps)
        if layer.get("mlp"):
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {layer['mlp']['kind']!r}")
            f = dense_ff(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
            x = x + rms_norm(f, w[p + "norm2b"], eps)
        if side:
            x = x + token_side(x, tok, w, p + "side.", i, int(side["dim"]), eps)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
