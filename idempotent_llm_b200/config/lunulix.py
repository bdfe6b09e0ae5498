"""Typed configuration of the Lunulix decoder, read from its config.json.

A Lunulix model is a list of layers.  Every layer norms its mixer's input and output, optionally does the
same around a dense gated feed-forward (gelu, tanh form), and ends with a small input that depends on the
token itself.  The one mixer there is, ``parallel``, runs two mixers on the same input and adds them with
constant weights: *left*, a grouped-query attention with short causal filters on q, k and v, a rotation of
part of each head with wavelength-dependent frequency scaling, a learned sink in the softmax and a sigmoid
output gate; *right*, a selective state-space mixer with scalar decay per head.

config.json keys (every size and every constant that differs between models is read from here):

    architecture            "Lunulix"
    vocab, width
    embedding.scale
    norm.eps
    token_side.dim          (absent or null: no token side input)
    layers[i].type          "parallel"
    layers[i].mixer.left    heads, kv_heads, dim, vdim, scale, conv (taps), rot {base, dims, scaling {factor,
                            low, high, original}}
    layers[i].mixer.right   heads, vdim, state, groups, conv (taps), norm_groups
    layers[i].mixer.left_scale, right_scale
    layers[i].mlp           null, or {kind: "dense", ff}

Tensor names: ``embed``, ``side.embed``, ``final.norm``, ``head``; layer i's start with ``l<i>.``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional, Tuple

from .specs import (ConfigError, GatedMLPNames, GatedMLPSpec, MixerBranch, ModelSpec, NormSpec, ParallelMixerSpec,
                    RotarySpec, SandwichLayerSpec, SinkAttentionSpec, SSDSpec, TokenSideSpec, WavelengthScaling,
                    default_schedule)

ARCHITECTURE = "Lunulix"
MAX_POSITIONS = 1 << 24          # the design sets no limit of its own; positions are 32-bit integers

MLP_NAMES = GatedMLPNames(gate="mlp.gate", up="mlp.up", down="mlp.down")


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where}: required key '{key}' is missing")
    return d[key]


def _pos_int(d, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or int(v) != v or int(v) <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return int(v)


@dataclass(frozen=True)
class LeftConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int                                   # taps; 1 = no filter
    rot_base: Optional[float]                   # None: no rotation
    rot_dims: int
    rot_scaling: Optional[Tuple[float, float, float, float]]    # factor, low, high, original

    @classmethod
    def from_dict(cls, d, where):
        rot = d.get("rot")
        base, dims, scaling = None, 0, None
        if rot:
            base, dims = float(_need(rot, "base", where + ".rot")), _pos_int(rot, "dims", where + ".rot")
            sc = rot.get("scaling")
            if sc:
                scaling = tuple(float(_need(sc, k, where + ".rot.scaling")) for k in ("factor", "low", "high", "original"))
        c = cls(heads=_pos_int(d, "heads", where), kv_heads=_pos_int(d, "kv_heads", where),
                dim=_pos_int(d, "dim", where), vdim=_pos_int(d, "vdim", where),
                scale=float(_need(d, "scale", where)), conv=int(d.get("conv") or 1),
                rot_base=base, rot_dims=dims, rot_scaling=scaling)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: heads={c.heads} is no multiple of kv_heads={c.kv_heads}")
        if c.rot_dims % 2 or c.rot_dims > c.dim:
            raise ConfigError(f"config.json: {where}.rot.dims={c.rot_dims} must be even and at most dim={c.dim}")
        if c.rot_base is not None and c.rot_base <= 0:
            raise ConfigError(f"config.json: {where}.rot.base must be positive")
        if scaling is not None and (scaling[0] <= 0 or scaling[2] == scaling[1] or scaling[3] <= 0):
            raise ConfigError(f"config.json: {where}.rot.scaling={scaling} cannot be applied")
        if c.conv < 1:
            raise ConfigError(f"config.json: {where}.conv={c.conv} must be at least 1")
        return c


@dataclass(frozen=True)
class RightConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, d, where):
        c = cls(heads=_pos_int(d, "heads", where), vdim=_pos_int(d, "vdim", where), state=_pos_int(d, "state", where),
                groups=_pos_int(d, "groups", where), conv=int(d.get("conv") or 1),
                norm_groups=int(d.get("norm_groups") or 1))
        if c.heads % c.groups:
            raise ConfigError(f"config.json: {where}: heads={c.heads} is no multiple of groups={c.groups}")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"config.json: {where}: heads * vdim = {c.heads * c.vdim} is no multiple of "
                              f"norm_groups={c.norm_groups}")
        if c.conv < 1:
            raise ConfigError(f"config.json: {where}.conv={c.conv} must be at least 1")
        return c


@dataclass(frozen=True)
class LunulixLayer:
    left: LeftConfig
    right: RightConfig
    left_scale: float
    right_scale: float
    ff: Optional[int]                           # None: the layer has no feed-forward


@dataclass(frozen=True)
class LunulixConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    token_side_dim: Optional[int]
    layers: Tuple[LunulixLayer, ...]
    raw: dict = None                            # config.json as read (written back unchanged)
    architecture: str = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, d: dict) -> "LunulixConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != ARCHITECTURE:
            raise ConfigError(f"config.json: architecture={name!r}, expected {ARCHITECTURE!r}")
        layers = []
        for i, L in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]"
            if _need(L, "type", where) != "parallel":
                raise ConfigError(f"config.json: {where}.type={L['type']!r}; the design has 'parallel'")
            m = _need(L, "mixer", where)
            mlp = L.get("mlp")
            if mlp is not None and _need(mlp, "kind", where + ".mlp") != "dense":
                raise ConfigError(f"config.json: {where}.mlp.kind={mlp['kind']!r}; the design has 'dense'")
            layers.append(LunulixLayer(
                left=LeftConfig.from_dict(_need(m, "left", where + ".mixer"), where + ".mixer.left"),
                right=RightConfig.from_dict(_need(m, "right", where + ".mixer"), where + ".mixer.right"),
                left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)),
                ff=None if mlp is None else _pos_int(mlp, "ff", where + ".mlp")))
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        side = d.get("token_side")
        emb = d.get("embedding") or {}
        cfg = cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"),
                  embedding_scale=float(emb.get("scale", 1.0)),
                  norm_eps=float(_need(_need(d, "norm", "config"), "eps", "norm")),
                  token_side_dim=None if not side else _pos_int(side, "dim", "token_side"),
                  layers=tuple(layers), raw=copy.deepcopy(d))
        if not cfg.norm_eps >= 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        return cfg

    # ----------------------------------------------------------------- write
    def to_dict(self) -> dict:
        d = copy.deepcopy(self.raw)
        d.setdefault("architecture", ARCHITECTURE)
        return d

    # ------------------------------------------------------------ translation
    def to_model_spec(self) -> ModelSpec:
        eps, W = self.norm_eps, self.width

        def norm(name):
            return NormSpec(size=W, eps=eps, weight=name)

        side_width = (self.token_side_dim or 0) * len(self.layers)
        specs = []
        for i, L in enumerate(self.layers):
            l, r = L.left, L.right
            rot = None
            if l.rot_base is not None and l.rot_dims:
                rot = RotarySpec(theta=l.rot_base, dim=l.rot_dims, max_positions=MAX_POSITIONS, variant="half_partial",
                                 scaling=None if l.rot_scaling is None else WavelengthScaling(*l.rot_scaling))
            left = SinkAttentionSpec(hidden=W, n_heads=l.heads, n_kv_heads=l.kv_heads, key_dim=l.dim, value_dim=l.vdim,
                                     softmax_scale=l.scale, conv_taps=l.conv, position=rot, sink=True, gate=True)
            right = SSDSpec(hidden=W, heads=r.heads, head_dim=r.vdim, state=r.state, groups=r.groups,
                            conv_taps=r.conv, norm_groups=r.norm_groups, norm_eps=eps)
            mixer = ParallelMixerSpec(hidden=W, prefix="mix.", branches=(
                MixerBranch(left, "left.", L.left_scale), MixerBranch(right, "right.", L.right_scale)))
            ff = None if L.ff is None else GatedMLPSpec(hidden=W, intermediate=L.ff, names=MLP_NAMES,
                                                        activation="gelu_tanh")
            side = None
            if self.token_side_dim:
                side = TokenSideSpec(hidden=W, dim=self.token_side_dim, col0=i * self.token_side_dim,
                                     vocab_size=self.vocab, table_width=side_width, eps=eps, table="side.embed")
            specs.append(SandwichLayerSpec(
                prefix=f"l{i}.", mixer=mixer, mixer_norm=norm("norm1"), mixer_post_norm=norm("norm1b"),
                feed_forward=ff, feed_forward_norm=None if ff is None else norm("norm2"),
                feed_forward_post_norm=None if ff is None else norm("norm2b"), token_side=side))
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden=W, layers=tuple(specs),
            schedule=default_schedule(len(specs)), final_norm=norm("norm"), tie_embeddings=False,
            max_positions=MAX_POSITIONS, embed_name="embed", final_norm_prefix="final.", head_name="head",
            embed_scale=self.embedding_scale)
