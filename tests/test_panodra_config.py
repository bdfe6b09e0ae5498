"""The Panodra configuration, its translation into specs, what its parts declare and ask of the cache, and the
plain implementation's mechanisms against closed forms of their own (CPU)."""

import json
import math
import os

import pytest
import torch

import helpers
import plain_panodra as plain
from idempotent_llm_b200.config import (ConfigError, DenseMLPSpec, DyTNormSpec, LatentAttentionSpec, PanodraConfig, RampScaling,
                                        RotarySpec, TableExpertsSpec)
from idempotent_llm_b200.engine.assembly import cache_needs, declare_weights
from idempotent_llm_b200.registry import read_config, registered_architectures

F64 = torch.float64


def test_every_key_is_read_per_layer():
    raw = helpers.PANODRA["A"]()
    cfg = PanodraConfig.from_dict(raw)
    assert "Panodra" in registered_architectures()
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.logit_scale, cfg.logit_softcap, cfg.loop) == (97, 64, 1e-5, 0.7, 12.0, (1, 3, 3))
    a, b, c = cfg.layers
    assert (a.mixer.sink, a.mixer.heads, a.mixer.dim, a.mixer.rot_dim, a.mixer.vdim, a.mixer.kv_rank) == (False, 3, 16, 8, 24, 40)
    assert a.mixer.rot_scaling is None and (a.mlp.kind, a.mlp.ff) == ("dense", 72)
    assert b.mixer.sink and b.mixer.rot_scaling == (8.0, 64.0, 8.0, 1.0) and (b.mlp.kind, b.mlp.ff, b.mlp.experts, b.mlp.top) == ("moe", 24, 5, 3)
    assert c.mixer.sink and c.mlp is None
    assert cfg.to_dict() == dict(raw)
    spec = cfg.to_model_spec()
    m = spec.layers[1].mixer
    assert isinstance(m, LatentAttentionSpec) and m.sink and (m.plain_dim, m.rot_dim, m.value_dim, m.kv_rank) == (8, 16, 8, 24)
    assert m.softmax_scale == 0.35 and m.eps == 1e-5 and m.position.variant == "interleaved" and m.position.dim == 16
    assert m.position.scaling == RampScaling(8.0, 64.0, 8.0, 1.0) and spec.layers[0].mixer.position.scaling is None
    assert isinstance(spec.layers[0].feed_forward, DenseMLPSpec) and spec.layers[0].feed_forward.activation == "relu2"
    ff = spec.layers[1].feed_forward
    assert isinstance(ff, TableExpertsSpec) and (ff.n_experts, ff.top, ff.intermediate, ff.vocab_size) == (5, 3, 24, 97)
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    assert isinstance(spec.final_norm, DyTNormSpec) and spec.tie_embeddings
    assert (spec.logit_scale, spec.logit_softcap, spec.mix_in_name) == (0.7, 12.0, "loop.in")


def test_the_order_of_layers_with_and_without_a_loop():
    spec = PanodraConfig.from_dict(helpers.PANODRA["A"]()).to_model_spec()
    got = [(e.layer, e.mix_in) for e in spec.schedule]
    assert got == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False)]
    assert [e.cache for e in spec.schedule] == list(range(7))             # every run has a cache entry of its own
    assert got == plain.layer_order(helpers.PANODRA["A"]())
    flat = PanodraConfig.from_dict(helpers.PANODRA["B"]()).to_model_spec()
    assert [(e.layer, e.mix_in) for e in flat.schedule] == [(0, False)] and flat.mix_in_name is None
    assert (flat.logit_scale, flat.logit_softcap) == (1.0, None)
    once = helpers.PANODRA["A"](); once["loop"] = dict(start=0, stop=3, times=1)
    assert [(e.layer, e.mix_in) for e in PanodraConfig.from_dict(once).to_model_spec().schedule] == [(0, True), (1, False), (2, False)]


def test_declared_tensors_and_what_the_mixer_keeps():
    spec = PanodraConfig.from_dict(helpers.PANODRA["A"]()).to_model_spec()
    d = {t.name: t for t in declare_weights(spec)}
    assert d["embed"].shape == (97, 64) and d["loop.in"].shape == (64, 128) and d["head"].optional
    assert d["l0.mix.q"].shape == (3 * 24, 64) and d["l0.mix.dkv"].shape == (48, 64) and d["l0.mix.dkv.norm"].shape == (40,)
    assert d["l0.mix.uk"].shape == (48, 40) and d["l0.mix.uv"].shape == (72, 40) and d["l0.mix.o"].shape == (64, 72)
    assert "l0.mix.sink" not in d and d["l1.mix.sink"].shape == (2,)
    assert d["l0.norm1.alpha"].shape == () and d["l0.norm1.b"].shape == (64,) and d["final.norm.alpha"].shape == ()
    assert d["l0.mlp.up"].shape == (72, 64) and d["l0.mlp.down"].shape == (64, 72)
    t = d["l1.mlp.table"]
    assert t.shape == (97, 3) and t.integer and t.high == 5
    assert d["l1.mlp.e4.gate"].shape == (24, 64) and d["l1.mlp.e4.down"].shape == (64, 24) and "l1.mlp.e5.gate" not in d
    assert "l2.norm2" not in d and "l2.mlp.up" not in d
    needs = cache_needs(spec)
    assert sorted(needs) == list(range(7))
    assert needs[0].key_row() == (1, 48) and needs[0].value_row() == (1, 0) and needs[0].kind == "full"     # one row per token
    assert needs[1].key_row() == needs[3].key_row() == (1, 40)


def test_refusals_name_the_key():
    for change, word in [(lambda c: c["layers"][0].update(type="attention"), "type"),
                         (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "kind"),
                         (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "top"),
                         (lambda c: c.update(loop=dict(start=2, stop=1, times=2)), "loop"),
                         (lambda c: c.update(logit_softcap=-1.0), "softcap"),
                         (lambda c: c.pop("width"), "width")]:
        c = helpers.PANODRA["A"]()
        change(c)
        with pytest.raises(ConfigError, match=word):
            PanodraConfig.from_dict(c)


def test_a_random_folder_is_loaded_by_name(tmp_path):
    from idempotent_llm_b200.weights import load_weights
    d = helpers.make_panodra_dir(helpers.PANODRA["A"](), str(tmp_path), seed=3)
    arch, cfg = read_config(d)
    assert arch.name == "Panodra"
    w = load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")
    table = w["l1.mlp.table"]
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 5
    assert all(len(set(row)) == 3 for row in table.tolist())               # a row's experts differ
    assert w["l0.norm1.alpha"].shape == () and 0.0 < float(w["l0.norm1.alpha"]) < 1.0
    # an integer table where a floating-point tensor is declared is refused
    from idempotent_llm_b200.weights import SafetensorsFile, WeightError, write_safetensors
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = [(n, f.get(n).clone().float() if n == "l1.mlp.table" else f.get(n).clone()) for n in f.names()]
    del f
    write_safetensors(path, tensors)
    with pytest.raises(WeightError, match="l1.mlp.table"):
        load_weights(d, declare_weights(cfg.to_model_spec()), "cpu")


# ----------------------------------------------------------------------------- the plain mechanisms
def test_frequencies_along_the_ramp_take_every_branch():
    from idempotent_llm_b200.parts.rotary import frequencies, magnitude
    rot = dict(base=1e4, dims=32, scaling=dict(factor=8.0, original=64, fast=8.0, slow=1.0))
    f, mag = plain.rotary_frequencies(rot)
    raw, one = plain.rotary_frequencies(dict(base=1e4, dims=32))
    assert one == 1.0 and abs(mag - (0.1 * math.log(8.0) + 1.0)) < 1e-15
    kept, slowed = (f == raw), ((f - raw / 8.0).abs() < 1e-18)
    assert kept[0] and slowed[-1] and (~kept & ~slowed).any()
    # by hand: lo = floor(32 ln(64 / 16 pi) / (2 ln 1e4)) = 0, hi = ceil(32 ln(64 / 2 pi) / (2 ln 1e4)) = 5
    ramp = torch.clamp(torch.arange(16, dtype=F64) / 5.0, 0, 1)
    assert (f - (raw / 8.0 * ramp + raw * (1 - ramp))).abs().max() < 1e-18
    spec = RotarySpec(theta=1e4, dim=32, max_positions=1 << 20, variant="interleaved", scaling=RampScaling(8.0, 64.0, 8.0, 1.0))
    assert (frequencies(spec) - f).abs().max() < 1e-15 and abs(magnitude(spec) - mag) < 1e-15
    # borders that meet: the ramp's width is floored at 0.001, a step from kept to slowed
    g, _ = plain.rotary_frequencies(dict(base=1e4, dims=8, scaling=dict(factor=2.0, original=1000, fast=3.0, slow=3.0)))
    spec = RotarySpec(theta=1e4, dim=8, max_positions=1 << 20, variant="interleaved", scaling=RampScaling(2.0, 1000.0, 3.0, 3.0))
    assert (frequencies(spec) - g).abs().max() < 1e-15


def test_neighbours_turn_like_complex_numbers():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 3, 8, generator=g, dtype=F64)
    f, mag = torch.tensor([1.0, 0.3, 0.05, 0.001], dtype=F64), 1.2
    pos = torch.tensor([0, 1, 7, 100, 1000])
    got = plain.rotate_pairs(x, pos, f, mag)
    z = torch.view_as_complex(x.reshape(5, 3, 4, 2).contiguous()) * torch.polar(torch.full((5, 1, 4), mag, dtype=F64),
                                                                                 (pos[:, None].double() * f)[:, None, :])
    assert (got - torch.view_as_real(z).reshape(5, 3, 8)).abs().max() < 1e-12
    assert torch.equal(plain.rotate_pairs(x[:1], pos[:1], f, 1.0), x[:1])          # position 0 turns nothing


def _mixer_weights(m, width, seed, sink):
    g = torch.Generator().manual_seed(seed)
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    w = {"M.q": torch.randn(H * (dn + dr), width, generator=g, dtype=F64) * 0.3,
         "M.dkv": torch.randn(R + dr, width, generator=g, dtype=F64) * 0.3, "M.dkv.norm": 1 + 0.1 * torch.randn(R, generator=g, dtype=F64),
         "M.uk": torch.randn(H * dn, R, generator=g, dtype=F64) * 0.3, "M.uv": torch.randn(H * dv, R, generator=g, dtype=F64) * 0.3,
         "M.o": torch.randn(width, H * dv, generator=g, dtype=F64) * 0.3}
    if sink:
        w["M.sink"] = torch.randn(H, generator=g, dtype=F64)
    return w


def test_the_sink_is_a_key_with_no_value_and_a_far_sink_is_no_sink():
    m = helpers.panodra_layer(sink=True, heads=2, dim=4, rot_dim=4, vdim=6, kv_rank=8)["mixer"]
    w = _mixer_weights(m, 12, 1, True)
    h = torch.randn(9, 12, generator=torch.Generator().manual_seed(2), dtype=F64)
    with_sink = plain.latent_attention(h, m, w, "M.", 1e-6)
    none = {k: v for k, v in w.items() if k != "M.sink"}
    far = dict(w); far["M.sink"] = torch.full((2,), -80.0, dtype=F64)
    assert (plain.latent_attention(h, m, far, "M.", 1e-6) - plain.latent_attention(h, m, none, "M.", 1e-6)).abs().max() < 1e-12
    assert (with_sink - plain.latent_attention(h, m, none, "M.", 1e-6)).abs().max() > 1e-3
    # the first token sees itself and the sink: its output is the no-sink output times 1 / (1 + exp(sink - s_00)) per head
    big = dict(w); big["M.sink"] = torch.full((2,), 80.0, dtype=F64)
    assert plain.latent_attention(h, m, big, "M.", 1e-6).abs().max() < 1e-12         # a sink far above takes all the weight


def test_the_latent_form_equals_keys_and_values_per_head():
    """Scores and values written out per head from the latent equal the same sums taken in the latent's space."""
    m = helpers.panodra_layer(heads=3, dim=6, rot_dim=4, vdim=5, kv_rank=7, scale=0.4)["mixer"]
    w = _mixer_weights(m, 10, 3, False)
    h = torch.randn(11, 10, generator=torch.Generator().manual_seed(4), dtype=F64)
    want = plain.latent_attention(h, m, w, "M.", 1e-5)
    T, H, dn, dr, dv, R = 11, 3, 6, 4, 5, 7
    pos = torch.arange(T)
    f, mag = plain.rotary_frequencies(m["rot"])
    q = (h @ w["M.q"].T).reshape(T, H, dn + dr)
    down = h @ w["M.dkv"].T
    c = plain.unit_rms(down[:, :R], w["M.dkv.norm"], 1e-5)
    rows = torch.cat([c, plain.rotate_pairs(down[:, R:], pos, f, mag)], dim=1)
    qa = torch.cat([torch.einsum("thd,hdr->thr", q[..., :dn], w["M.uk"].reshape(H, dn, R)),
                    plain.rotate_pairs(q[..., dn:], pos, f, mag)], dim=-1)
    s = torch.einsum("thr,jr->htj", qa, rows) * 0.4
    s = s.masked_fill(~(pos[None, :] <= pos[:, None])[None], -math.inf)
    ctx = torch.einsum("htj,jr->thr", torch.softmax(s, dim=-1), c)
    o = torch.einsum("thr,hvr->thv", ctx, w["M.uv"].reshape(H, dv, R)).reshape(T, H * dv) @ w["M.o"].T
    assert (o - want).abs().max() < 1e-12


def test_table_experts_against_a_dense_sum_and_the_norm_by_hand():
    g = torch.Generator().manual_seed(5)
    W, ff, E, top, V = 6, 4, 3, 2, 7
    w = {"F.table": torch.tensor([[0, 1], [2, 0], [1, 2], [0, 2], [2, 1], [1, 0], [0, 1]], dtype=torch.int32)}
    for e in range(E):
        w[f"F.e{e}.gate"], w[f"F.e{e}.up"] = torch.randn(ff, W, generator=g, dtype=F64), torch.randn(ff, W, generator=g, dtype=F64)
        w[f"F.e{e}.down"] = torch.randn(W, ff, generator=g, dtype=F64)
    h = torch.randn(5, W, generator=g, dtype=F64)
    toks = [3, 0, 6, 4, 3]
    got = plain.table_experts(h, toks, dict(router=dict(top=top)), w, "F.")
    every = torch.stack([(plain.silu(h @ w[f"F.e{e}.gate"].T) * (h @ w[f"F.e{e}.up"].T)) @ w[f"F.e{e}.down"].T for e in range(E)])
    use = torch.zeros(5, E, dtype=F64)
    for t, tok in enumerate(toks):
        use[t, w["F.table"][tok].long()] = 1.0 / top
    assert (got - torch.einsum("te,etw->tw", use, every)).abs().max() < 1e-12
    x = torch.tensor([[-2.0, 0.0, 0.5]], dtype=F64)
    assert (plain.dyt(x, 0.5, torch.tensor([2.0, 1.0, 1.0], dtype=F64), torch.tensor([0.0, 3.0, 0.0], dtype=F64))
            - torch.tensor([[2 * math.tanh(-1.0), 3.0, math.tanh(0.25)]], dtype=F64)).abs().max() < 1e-15
    y = plain.dense_ff(torch.tensor([[1.0, -1.0]], dtype=F64), {"D.up": torch.tensor([[2.0, 0.0], [0.0, 3.0]], dtype=F64),
                                                               "D.down": torch.tensor([[1.0, 1.0]], dtype=F64)}, "D.")
    assert float(y) == 4.0                                                  # relu(2)^2 + relu(-3)^2


def test_the_plain_model_runs_every_configuration(tmp_path):
    for name in ("A", "B", "C"):
        d = helpers.make_panodra_dir(helpers.PANODRA[name](), str(tmp_path / name), seed=2)
        cfg, w = helpers.read_model_dir(d)
        toks = helpers.rand_ids(12, cfg["vocab"], 1)
        streams = []
        lg = plain.forward(cfg, w, toks, streams)
        assert lg.shape == (12, cfg["vocab"]) and torch.isfinite(lg).all() and len(streams) == len(plain.layer_order(cfg))
        if cfg.get("logit_softcap"):
            assert float(lg.abs().max()) < cfg["logit_softcap"]
        # causal: a token's logits do not depend on what follows
        assert (plain.forward(cfg, w, toks[:7]) - lg[:7]).abs().max() < 1e-9
