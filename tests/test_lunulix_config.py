"""Lunulix on the CPU: configuration and registry, the specs it translates to, declared tensors, what the
parallel mixer asks of the cache, random model folders, and the plain implementation's mechanisms against
closed forms of their own."""

import copy
import json
import math
import os

import pytest
import torch

import helpers
import plain_lunulix as plain
from idempotent_llm_b200 import registry
from idempotent_llm_b200.config import ConfigError, LunulixConfig
from idempotent_llm_b200.config.presets import preset
from idempotent_llm_b200.engine.assembly import cache_needs, declare_weights

F64 = torch.float64


def test_every_size_and_constant_is_read_per_layer():
    cfg = LunulixConfig.from_dict(helpers.LUNULIX["P"]())
    a, b = cfg.layers
    for side in ("left", "right"):
        for k, va in vars(getattr(a, side)).items():
            assert va != getattr(getattr(b, side), k) or k in ("rot_base", "kv_heads"), f"the two layers share {side}.{k}"
    assert (a.left_scale, a.right_scale, a.ff) == (0.7, 1.3, 40) and (b.left_scale, b.right_scale, b.ff) == (1.0, 0.5, None)
    assert a.left.rot_scaling == (4.0, 1.0, 4.0, 64.0) and b.left.rot_scaling is None
    assert (cfg.vocab, cfg.width, cfg.embedding_scale, cfg.norm_eps, cfg.token_side_dim) == (97, 32, 3.0, 1e-5, 8)
    spec = cfg.to_model_spec()
    l0, l1 = spec.layers
    assert l0.kind == "sandwich" and l0.mixer.kind == "parallel"
    left, right = (br.mixer for br in l0.mixer.branches)
    assert (left.n_heads, left.n_kv_heads, left.key_dim, left.value_dim, left.conv_taps) == (4, 2, 16, 24, 3)
    assert left.position.dim == 8 and left.position.scaling.original == 64
    assert (right.heads, right.head_dim, right.state, right.groups, right.conv_taps, right.norm_groups) == (3, 8, 12, 1, 4, 2)
    assert l1.feed_forward is None and l1.feed_forward_norm is None and l0.feed_forward.activation == "gelu_tanh"
    assert l1.token_side.col0 == 8 and l1.token_side.table_width == 16 and spec.embed_scale == 3.0
    assert l1.mixer.branches[0].mixer.position.scaling is None


def test_optional_parts_may_be_absent():
    cfg = LunulixConfig.from_dict(helpers.LUNULIX["Q"]())
    spec = cfg.to_model_spec()
    left = spec.layers[0].mixer.branches[0].mixer
    assert left.position is None and left.conv_taps == 1 and spec.layers[0].token_side is None and spec.embed_scale == 1.0
    names = {d.name for d in declare_weights(spec)}
    assert "side.embed" not in names and "l0.mix.left.q.conv" not in names and "l0.mix.left.sink" in names


def test_declared_tensors_and_shapes():
    spec = LunulixConfig.from_dict(helpers.LUNULIX["P"]()).to_model_spec()
    d = {x.name: x.shape for x in declare_weights(spec)}
    assert d["embed"] == (97, 32) and d["head"] == (97, 32) and d["final.norm"] == (32,) and d["side.embed"] == (97, 16)
    assert d["l0.mix.left.q"] == (64, 32) and d["l0.mix.left.k"] == (32, 32) and d["l0.mix.left.v"] == (48, 32)
    assert d["l0.mix.left.q.conv"] == (64, 3) and d["l0.mix.left.v.conv"] == (48, 3) and d["l0.mix.left.sink"] == (4,)
    assert d["l0.mix.left.g"] == (96, 32) and d["l0.mix.left.o"] == (32, 96)
    assert d["l0.mix.right.in"] == (2 * 24 + 2 * 12 + 3, 32) and d["l0.mix.right.conv"] == (48, 4) and d["l0.mix.right.conv.b"] == (48,)
    assert d["l0.mix.right.norm"] == (24,) and d["l0.mix.right.o"] == (32, 24) and d["l0.mix.right.A_log"] == (3,)
    assert d["l0.mlp.gate"] == (40, 32) and d["l0.side.gate"] == (8, 32) and d["l0.side.proj"] == (32, 8)
    assert "l1.mlp.gate" not in d and "l1.norm2" not in d and "l1.norm1b" in d and "l1.side.norm" in d


def test_the_parallel_mixer_asks_for_keys_of_one_branch_and_state_of_both():
    spec = LunulixConfig.from_dict(helpers.LUNULIX["P"]()).to_model_spec()
    needs = cache_needs(spec)
    n0, n1 = needs[0], needs[1]
    assert n0.kind == "full" and n0.key_row() == (2, 16) and n0.value_row() == (2, 24)
    assert n0.state_shape == (2 * (6 * 16 + 2 * 24) + 3 * 48 + 3 * 12 * 8,)
    assert n1.key_row() == (2, 24) and n1.value_row() == (2, 16)
    assert n0.group_key() != n1.group_key()          # unlike layers get storage of their own


def test_registry_reads_one_architecture_name(tmp_path):
    d = helpers.LUNULIX["Q"]()
    with open(tmp_path / "config.json", "w") as f:
        json.dump(d, f)
    arch, cfg = registry.read_config(str(tmp_path))
    assert arch.name == "Lunulix" and isinstance(cfg, LunulixConfig) and cfg.to_dict() == d
    assert "Lunulix" in registry.registered_architectures()
    assert preset("lunulix-tiny").width == 96


@pytest.mark.parametrize("path,value,match", [
    (("layers", 0, "type"), "serial", "type"),
    (("layers", 0, "mlp", "kind"), "routed", "dense"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "multiple"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 18, "dims"),
    (("layers", 0, "mixer", "right", "norm_groups"), 5, "norm_groups"),
    (("layers", 0, "mixer", "right", "groups"), 2, "groups"),
    (("norm",), None, "norm"),
    (("vocab",), 0, "vocab"),
])
def test_bad_values_are_refused_by_name(path, value, match):
    d = copy.deepcopy(helpers.LUNULIX["P"]())
    at = d
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=match):
        LunulixConfig.from_dict(d)


def test_a_random_model_folder_loads_by_name(tmp_path):
    from idempotent_llm_b200.weights import load_weights
    d = helpers.make_lunulix_dir(helpers.LUNULIX["P"](), str(tmp_path), seed=4)
    arch, cfg = registry.read_config(d)
    w = load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    assert w["l1.mix.right.conv"].shape == (4 * 12 + 2 * 2 * 10, 3) and w["side.embed"].dtype == torch.bfloat16
    assert float(w["l0.mix.left.q.conv"].float().std()) > 0.3          # filters are of order one, not of the matrices' size


# ------------------------------------------------------------------ the plain implementation against closed forms
def test_plain_filter_is_a_causal_correlation():
    g = torch.Generator().manual_seed(0)
    u, w = torch.randn(11, 5, generator=g, dtype=F64), torch.randn(5, 3, generator=g, dtype=F64)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (2, 0)), w[:, None, :], groups=5)[0].T
    assert (plain.causal_conv(u, w) - want).abs().max() < 1e-12
    assert (plain.causal_conv(u, w)[0] - u[0] * w[:, 2]).abs().max() < 1e-12         # the last tap is the current token's


def test_plain_recurrence_equals_its_unrolled_sum():
    """y_t = sum_{s <= t} exp(-a (dt_(s+1) + .. + dt_t)) dt_s (C_t . B_s) x_s + D x_t."""
    g = torch.Generator().manual_seed(1)
    T, H, P, G, N = 9, 2, 3, 1, 4
    x, dt = torch.randn(T, H, P, generator=g, dtype=F64), torch.rand(T, H, generator=g, dtype=F64)
    B, C = torch.randn(T, G, N, generator=g, dtype=F64), torch.randn(T, G, N, generator=g, dtype=F64)
    a, D = torch.tensor([0.3, 1.7], dtype=F64), torch.tensor([0.5, -1.0], dtype=F64)
    got = plain.ssd_scan(x, dt, a, B, C, D)
    for h in range(H):
        cum = torch.cumsum(dt[:, h], 0)
        for t in range(T):
            want = D[h] * x[t, h]
            for s in range(t + 1):
                want = want + torch.exp(-a[h] * (cum[t] - cum[s])) * dt[s, h] * (C[t, 0] @ B[s, 0]) * x[s, h]
            assert (got[t, h] - want).abs().max() < 1e-12


def test_plain_sink_only_lowers_the_weights():
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(6, 2, 4, generator=g, dtype=F64) for _ in range(3))
    none = plain.sink_attention(q, k[:, :1], v[:, :1], 0.5, None)
    low = plain.sink_attention(q, k[:, :1], v[:, :1], 0.5, torch.tensor([-50.0, -50.0], dtype=F64))
    high = plain.sink_attention(q, k[:, :1], v[:, :1], 0.5, torch.tensor([50.0, 0.0], dtype=F64))
    assert (none - low).abs().max() < 1e-12 and high[:, 0].abs().max() < 1e-12
    assert (none[0] - v[0, 0]).abs().max() < 1e-12                       # the first token sees itself only
    assert (high[0, 1] - v[0, 0] * math.exp(q[0, 1] @ k[0, 0] * 0.5) / (math.exp(q[0, 1] @ k[0, 0] * 0.5) + 1.0)).abs().max() < 1e-12


def test_plain_rotation_turns_pairs_half_apart_and_leaves_the_rest():
    f = plain.rotary_frequencies(dict(base=100.0, dims=4))
    assert torch.allclose(f, torch.tensor([1.0, 0.1], dtype=F64))
    x = torch.arange(6, dtype=F64).reshape(1, 1, 6) + 1.0
    y = plain.rotate(x, torch.tensor([3]), f)[0, 0]
    assert torch.allclose(y[4:], x[0, 0, 4:])
    assert abs(y[0] - (1.0 * math.cos(3.0) - 3.0 * math.sin(3.0))) < 1e-12 and abs(y[3] - (4.0 * math.cos(0.3) + 2.0 * math.sin(0.3))) < 1e-12
