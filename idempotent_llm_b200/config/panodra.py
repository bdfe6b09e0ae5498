"""Typed configuration of the Panodra decoder, read from its config.json.

A Panodra model is a list of pre-norm layers whose norm has no statistics (``tanh(alpha x) * w + b``).  Every
layer's mixer is an attention through a latent: a token keeps one normed vector of ``kv_rank`` numbers, from which
every head's unrotated keys and values are linear maps, and one rotated key part shared by all heads.  The two
mixer types differ in the softmax (``latent_attention``: a learned sink per head in the denominator;
``latent_attention_2``: the ordinary one) and both may scale their rotation's frequencies along a ramp.  A layer's
feed-forward is absent, dense (``down(relu(up x)^2)``) or a set of gated experts chosen by a table over token ids.
A stretch of layers may run several times in a row with the same weights, each pass with a cache of its own and
opened by a matrix that mixes the running stream with the embedding output.  The head is the embedding table;
logits are multiplied by a constant and capped softly.

config.json keys (every size and every constant that differs between models is read from here):

    architecture            "Panodra"
    vocab, width
    norm.eps                (the latent's root mean square)
    logit_scale, logit_softcap      (absent: 1 and no cap)
    loop                    absent or null, or {start, stop, times}
    layers[i].type          "latent_attention" | "latent_attention_2"
    layers[i].mixer         heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims, scaling {factor, original,
                            fast, slow}}
    layers[i].mlp           null, {kind: "dense", ff}, or {kind: "moe", expert {ff}, router {experts, top}}

Tensor names: ``embed``, ``loop.in``, ``final.norm`` (+ ``.alpha``, ``.b``); layer i's start with ``l<i>.``:
``norm1``, ``norm2`` (+ ``.alpha``, ``.b``), ``mix.q``, ``mix.dkv``, ``mix.dkv.norm``, ``mix.uk``, ``mix.uv``,
``mix.sink``, ``mix.o``, ``mlp.up``, ``mlp.down``, ``mlp.table``, ``mlp.e<k>.gate`` / ``up`` / ``down``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional, Tuple

from .specs import (ConfigError, DenseMLPNames, DenseMLPSpec, DyTNormSpec, LatentAttentionNames, LatentAttentionSpec, LayerSpec, ModelSpec, RampScaling,
                    RotarySpec, RunEntry, TableExpertsSpec)

ARCHITECTURE = "Panodra"
MAX_POSITIONS = 1 << 24          # the design sets no limit of its own; positions are 32-bit integers
MIXER_NAMES = LatentAttentionNames(q="mix.q", down="mix.dkv", down_norm="mix.dkv.norm", up_k="mix.uk", up_v="mix.uv", o="mix.o",
                                   sink="mix.sink")
DENSE_NAMES = DenseMLPNames(up="mlp.up", down="mlp.down")
MIXER_TYPES = {"latent_attention": True, "latent_attention_2": False}     # type -> a sink in the softmax


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
class PanodraMixer:
    sink: bool
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[Tuple[float, float, float, float]]     # factor, original, fast, slow

    @classmethod
    def from_dict(cls, kind: str, d, where):
        rot = _need(d, "rot", where)
        sc = rot.get("scaling")
        scaling = None
        if sc:
            scaling = tuple(float(_need(sc, k, where + ".rot.scaling")) for k in ("factor", "original", "fast", "slow"))
            if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
                raise ConfigError(f"config.json: {where}.rot.scaling={scaling} cannot be applied")
        m = cls(sink=MIXER_TYPES[kind], heads=_pos_int(d, "heads", where), dim=_pos_int(d, "dim", where),
                rot_dim=_pos_int(d, "rot_dim", where), vdim=_pos_int(d, "vdim", where),
                kv_rank=_pos_int(d, "kv_rank", where), scale=float(_need(d, "scale", where)),
                rot_base=float(_need(rot, "base", where + ".rot")), rot_dims=_pos_int(rot, "dims", where + ".rot"),
                rot_scaling=scaling)
        if m.rot_dims % 2 or m.rot_dims > m.rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims={m.rot_dims} must be even and at most rot_dim={m.rot_dim}")
        if m.rot_base <= 0 or (scaling is not None and m.rot_base == 1.0):
            raise ConfigError(f"config.json: {where}.rot.base={m.rot_base} cannot be used")
        return m


@dataclass(frozen=True)
class PanodraMLP:
    kind: str                   # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, d, where):
        kind = _need(d, "kind", where)
        if kind == "dense":
            return cls(kind="dense", ff=_pos_int(d, "ff", where))
        if kind == "moe":
            r = _need(d, "router", where)
            m = cls(kind="moe", ff=_pos_int(_need(d, "expert", where), "ff", where + ".expert"),
                    experts=_pos_int(r, "experts", where + ".router"), top=_pos_int(r, "top", where + ".router"))
            if m.top > m.experts:
                raise ConfigError(f"config.json: {where}.router: top={m.top} of {m.experts} experts")
            return m
        raise ConfigError(f"config.json: {where}.kind={kind!r}; the design has 'dense' and 'moe'")


@dataclass(frozen=True)
class PanodraLayer:
    mixer: PanodraMixer
    mlp: Optional[PanodraMLP]


@dataclass(frozen=True)
class PanodraConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    logit_softcap: Optional[float]
    loop: Optional[Tuple[int, int, int]]        # start, stop, times
    layers: Tuple[PanodraLayer, ...]
    raw: dict = None                            # config.json as read (written back unchanged)
    architecture: str = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, d: dict) -> "PanodraConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != ARCHITECTURE:
            raise ConfigError(f"config.json: architecture={name!r}, expected {ARCHITECTURE!r}")
        layers = []
        for i, L in enumerate(_need(d, "layers", "config")):
            where = f"layers[{i}]"
            kind = _need(L, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type={kind!r}; the design has {sorted(MIXER_TYPES)}")
            mlp = L.get("mlp")
            layers.append(PanodraLayer(mixer=PanodraMixer.from_dict(kind, _need(L, "mixer", where), where + ".mixer"),
                                       mlp=None if mlp is None else PanodraMLP.from_dict(mlp, where + ".mlp")))
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        loop = d.get("loop")
        if loop:
            loop = (int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")), _pos_int(loop, "times", "loop"))
            if not 0 <= loop[0] < loop[1] <= len(layers):
                raise ConfigError(f"config.json: loop {loop[0]}..{loop[1]} does not lie within {len(layers)} layers")
        cap = d.get("logit_softcap")
        cfg = cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"),
                  norm_eps=float(_need(_need(d, "norm", "config"), "eps", "norm")),
                  logit_scale=float(d.get("logit_scale", 1.0)), logit_softcap=None if not cap else float(cap),
                  loop=loop or None, layers=tuple(layers), raw=copy.deepcopy(d))
        if not cfg.norm_eps >= 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        if cfg.logit_softcap is not None and cfg.logit_softcap <= 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        return cfg

    # ----------------------------------------------------------------- write
    def to_dict(self) -> dict:
        d = copy.deepcopy(self.raw)
        d.setdefault("architecture", ARCHITECTURE)
        return d

    # ------------------------------------------------------------ translation
    def schedule(self) -> Tuple[RunEntry, ...]:
        """Layers before the loop once, the loop's layers ``times`` times (each run with a cache entry of its own, each
        pass opened by the mix with the embedding), the rest once."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(RunEntry(layer=i, cache=i) for i in range(n))
        a, b, times = self.loop
        order = [(i, False) for i in range(a)]
        for _ in range(times):
            order += [(i, i == a) for i in range(a, b)]
        order += [(i, False) for i in range(b, n)]
        return tuple(RunEntry(layer=i, cache=c, mix_in=m) for c, (i, m) in enumerate(order))

    def to_model_spec(self) -> ModelSpec:
        W = self.width
        specs = []
        for i, L in enumerate(self.layers):
            m = L.mixer
            rot = RotarySpec(theta=m.rot_base, dim=m.rot_dims, max_positions=MAX_POSITIONS, variant="interleaved",
                             scaling=None if m.rot_scaling is None else RampScaling(*m.rot_scaling))
            mixer = LatentAttentionSpec(hidden=W, n_heads=m.heads, plain_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim,
                                        kv_rank=m.kv_rank, softmax_scale=m.scale, eps=self.norm_eps, position=rot,
                                        sink=m.sink, names=MIXER_NAMES)
            ff = None
            if L.mlp is not None and L.mlp.kind == "dense":
                ff = DenseMLPSpec(hidden=W, intermediate=L.mlp.ff, activation="relu2", names=DENSE_NAMES)
            elif L.mlp is not None:
                ff = TableExpertsSpec(hidden=W, intermediate=L.mlp.ff, n_experts=L.mlp.experts, top=L.mlp.top,
                                      vocab_size=self.vocab, activation="silu", table="mlp.table", expert="mlp.e{}.")
            specs.append(LayerSpec(prefix=f"l{i}.", mixer=mixer, feed_forward=ff,
                                   mixer_norm=DyTNormSpec(size=W, weight="norm1"),
                                   feed_forward_norm=None if ff is None else DyTNormSpec(size=W, weight="norm2"),
                                   mixer_norm_prefix="", feed_forward_norm_prefix="", kind="prenorm"))
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden=W, layers=tuple(specs), schedule=self.schedule(),
            final_norm=DyTNormSpec(size=W, weight="norm"), tie_embeddings=True, max_positions=MAX_POSITIONS,
            embed_name="embed", final_norm_prefix="final.", head_name="head",
            mix_in_name="loop.in" if self.loop is not None else None,
            logit_scale=self.logit_scale, logit_softcap=self.logit_softcap)
