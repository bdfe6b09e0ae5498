"""The Lunulix decoder on the GPU against the plain implementation (``plain_lunulix.py``): every mechanism
alone, then whole models through the engine: prompts, token-by-token decoding, portions, unequal batches,
slots and pages used again, far keys and page borders, first tokens, long decoding, greedy generation, and
the trace replay program."""

import os

import pytest
import torch

import helpers
import plain_lunulix as plain
from idempotent_llm_b200 import api
from idempotent_llm_b200.cache import SequenceCache
from idempotent_llm_b200.config import (MixerBranch, ParallelMixerSpec, RotarySpec, SinkAttentionSpec, SSDSpec,
                                        WavelengthScaling)
from idempotent_llm_b200.engine.batch import context_from_packed, pack_step_host
from idempotent_llm_b200.parts import MIXERS, Runtime
from idempotent_llm_b200.weights import random_weights

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# against the 64-bit plain implementation, relative to the largest value: 32-bit arithmetic rounds at 6e-8 a few
# hundred times per layer and every norm behind a sublayer passes the error on at full size; bfloat16 rounds
# activations at 4e-3 a handful of times per layer.  A wrong mechanism shows at 1e-2 and above.
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
F64 = torch.float64


def _close(got, want, dtype):
    """32-bit: the largest difference, relative to the largest value.  bfloat16: the root mean square of the
    difference relative to that of the values, and a looser bound on the largest one: where a sublayer's output
    is small, the norm behind it enlarges the rounding of single tokens, which a mean absorbs and a maximum
    does not."""
    if dtype == "float32":
        return helpers.rel_err(got, want) < TOL[dtype]
    g, w = got.detach().double().cpu(), want.detach().double().cpu()
    rms = float((g - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt())
    return rms < TOL[dtype] and helpers.rel_err(got, want) < 0.25


def _rt(dtype):
    from idempotent_llm_b200.kernels import Kernels
    dev = torch.device("cuda:0")
    return Runtime(device=dev, dtype=DT[dtype], kernels=Kernels(DT[dtype], dev))


def _ctx(slots, starts, lens):
    packed, n, q_lens = pack_step_host(slots, starts, [[0] * L for L in lens])
    return context_from_packed(packed.cuda(), n, slots, q_lens, starts)


def _w64(w):
    return {k: v.double().cpu() for k, v in w.items()}


def _cuts(T, sizes):
    """(lo, hi) portions of 0 .. T with the given sizes in turn, the last one repeated."""
    out, lo, i = [], 0, 0
    while lo < T:
        n = sizes[min(i, len(sizes) - 1)]
        out.append((lo, min(T, lo + n)))
        lo, i = lo + n, i + 1
    return out


# ----------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("taps,bias,act", [(2, False, 0), (3, True, 1), (4, True, 1), (8, False, 0)])
def test_short_filter_with_state_in_portions(taps, bias, act):
    """The filter of a sequence fed in portions of 1, 2 and more tokens, next to a second sequence in the same
    steps, equals the filter of the whole; columns are a slice of a wider projection."""
    K = _rt("float32").kernels
    C, width, col0, T = 37, 50, 9, 23
    g = torch.Generator().manual_seed(taps)
    u = torch.randn(2, T, width, generator=g)
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g) if bias else None
    state = torch.zeros(4, (taps - 1) * C + 5, device="cuda")[:, 2:2 + (taps - 1) * C]      # a view: rows are strided
    got = [[], []]
    for lo, hi in _cuts(T, [1, 1, 2, 5, 1, 3, 1]):
        ctx = _ctx([3, 1], [lo, lo], [hi - lo, hi - lo])
        proj = torch.cat([u[0, lo:hi], u[1, lo:hi]]).contiguous().cuda()
        y = K.short_conv(proj, col0, C, w.cuda(), None if b is None else b.cuda(), act, state, ctx)
        if hi - lo > 1:
            K.conv_state_update(proj, col0, C, taps, state, ctx)
        got[0].append(y[:hi - lo].cpu())
        got[1].append(y[hi - lo:].cpu())
    for i in range(2):
        want = plain.causal_conv(u[i, :, col0:col0 + C].double(), w.double(), None if b is None else b.double())
        want = plain.silu(want) if act else want
        assert (torch.cat(got[i]).double() - want).abs().max() < 2e-5


def test_scaled_frequencies_in_all_three_ranges():
    """Short waves kept, long waves divided, a blend between; checked against the plain formula and by hand."""
    from idempotent_llm_b200.parts.rotary import frequencies
    spec = RotarySpec(theta=10000.0, dim=32, max_positions=1 << 20, variant="half_partial",
                      scaling=WavelengthScaling(factor=8.0, low=1.0, high=4.0, original=256.0))
    f = frequencies(spec)
    want = plain.rotary_frequencies(dict(base=10000.0, dims=32, scaling=dict(factor=8.0, low=1.0, high=4.0, original=256.0)))
    assert (f - want).abs().max() < 1e-15
    raw = plain.rotary_frequencies(dict(base=10000.0, dims=32))
    kept, divided = (f == raw), ((f - raw / 8.0).abs() < 1e-18)
    assert kept.any() and divided.any() and (~kept & ~divided).any()          # every branch is taken
    assert kept[0] and divided[-1]


def _sink_spec(**kw):
    base = dict(hidden=40, n_heads=6, n_kv_heads=2, key_dim=24, value_dim=40, softmax_scale=0.3, conv_taps=3,
                position=RotarySpec(3e4, 16, 1 << 20, variant="half_partial",
                                    scaling=WavelengthScaling(4.0, 1.0, 4.0, 64.0)), sink=True, gate=True)
    base.update(kw)
    return SinkAttentionSpec(**base)


def _plain_left_cfg(s):
    c = dict(heads=s.n_heads, kv_heads=s.n_kv_heads, dim=s.key_dim, vdim=s.value_dim, scale=s.softmax_scale)
    if s.conv_taps > 1:
        c["conv"] = s.conv_taps
    if s.position is not None:
        c["rot"] = dict(base=s.position.theta, dims=s.position.dim)
        if s.position.scaling is not None:
            sc = s.position.scaling
            c["rot"]["scaling"] = dict(factor=sc.factor, low=sc.low, high=sc.high, original=sc.original)
    return c


def _plain_left(x, w, s):
    """The plain attention side for a spec that may lack the gate or the sink."""
    w = dict(w)
    if not s.gate:                                   # sigmoid(large) = 1
        w["L.g"] = torch.zeros(s.n_heads * s.value_dim, s.hidden, dtype=F64)
        out = plain.left_mixer(x, w, "L.", _plain_left_cfg(s))
        return out * 2.0
    return plain.left_mixer(x, w, "L.", _plain_left_cfg(s))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", ["all", "bare", "whole_head", "wide_keys", "tensor_core_64", "tensor_core_128",
                                     "tensor_core_64_long"])
def test_sink_attention_alone_prompt_then_single_tokens(dtype, variant):
    """(Key and value rows of 64 or 128 elements take the tensor-core attention in bfloat16, which folds the sink
    behind the last run of keys; every other shape, and 32-bit, the general kernel.)"""
    spec = {"all": _sink_spec(),
            "tensor_core_64": _sink_spec(key_dim=64, value_dim=64, n_heads=4, n_kv_heads=2, softmax_scale=0.15,
                                         position=RotarySpec(3e4, 32, 1 << 20, variant="half_partial")),
            # (more than 512 keys: several runs of key blocks, folded through scratch, the sink behind the last)
            "tensor_core_64_long": _sink_spec(key_dim=64, value_dim=64, n_heads=4, n_kv_heads=1, softmax_scale=0.15,
                                              position=RotarySpec(3e4, 32, 1 << 20, variant="half_partial")),
            "tensor_core_128": _sink_spec(key_dim=128, value_dim=128, n_heads=3, n_kv_heads=1, softmax_scale=0.1, gate=False,
                                          position=RotarySpec(3e4, 128, 1 << 20, variant="half_partial")),
            "bare": _sink_spec(conv_taps=1, position=None, sink=False, gate=False, n_kv_heads=6),
            "whole_head": _sink_spec(position=RotarySpec(1e4, 24, 1 << 20, variant="half_partial"), conv_taps=2, n_kv_heads=1),
            "wide_keys": _sink_spec(key_dim=72, value_dim=8, n_heads=2, n_kv_heads=1,
                                    position=RotarySpec(5e5, 40, 1 << 20, variant="half_partial"))}[variant]
    rt = _rt(dtype)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "L."), 5, 0.25, dtype=DT[dtype], device="cuda")
    if spec.sink:
        w["L.sink"] = torch.tensor([2.5, -1.0, 0.5, 4.0, 0.0, 1.0][:spec.n_heads], device="cuda").to(DT[dtype])
    part = cls(spec, w, "L.", rt)
    need = cls.cache_need(spec)
    assert need.key_row() == (spec.n_kv_heads, spec.key_dim) and need.value_row() == (spec.n_kv_heads, spec.value_dim)
    T, pre = (1300, 1291) if variant.endswith("long") else (140, 131)
    cache = SequenceCache({0: need}, 64 * 24, DT[dtype], "cuda:0", max_seqs=2)
    slot = cache.alloc_slot()
    x = (torch.randn(T, spec.hidden, generator=torch.Generator().manual_seed(3)) * 1.5).to(DT[dtype])
    ref = _plain_left(x.double(), _w64(w), spec)
    outs = []
    for lo, hi in [(0, pre)] + [(i, i + 1) for i in range(pre, T)]:
        cache.reserve([(slot, hi)]); cache.flush()
        ctx = _ctx([slot], [lo], [hi - lo])
        outs.append(part.forward(x[lo:hi].contiguous().cuda(), ctx, cache.view(0), cache.state_of(0), True).sum(0))
        cache.set_length(slot, hi)
    assert helpers.rel_err(torch.cat(outs), ref) < TOL[dtype]


def test_the_sink_takes_weight_without_a_value():
    """With a sink far above every score the output vanishes; with one far below it is plain softmax attention."""
    spec = _sink_spec(conv_taps=1, position=None, gate=False, n_heads=2, n_kv_heads=1, key_dim=8, value_dim=8, hidden=16)
    rt = _rt("float32")
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "L."), 7, 0.3, dtype=torch.float32, device="cuda")
    x = torch.randn(9, 16, generator=torch.Generator().manual_seed(1))
    outs = {}
    for name, sink in (("high", 40.0), ("low", -40.0)):
        w["L.sink"] = torch.full((2,), sink, device="cuda")
        part = cls(spec, w, "L.", rt)
        cache = SequenceCache({0: cls.cache_need(spec)}, 64, torch.float32, "cuda:0", max_seqs=1)
        slot = cache.alloc_slot()
        cache.reserve([(slot, 9)]); cache.flush()
        outs[name] = part.forward(x.cuda(), _ctx([slot], [0], [9]), cache.view(0), None, True).sum(0).cpu()
    assert outs["high"].abs().max() < 1e-10
    no_sink = dict(_w64(w)); no_sink["L.sink"] = torch.full((2,), -1e9, dtype=F64); no_sink["L.g"] = torch.zeros(16, 16, dtype=F64)
    want = 2.0 * plain.left_mixer(x.double(), no_sink, "L.", _plain_left_cfg(spec))
    assert helpers.rel_err(outs["low"], want) < 1e-5


def _ssd_spec(**kw):
    base = dict(hidden=40, heads=3, head_dim=24, state=20, groups=1, conv_taps=4, norm_groups=4, norm_eps=1e-5)
    base.update(kw)
    return SSDSpec(**base)


def _plain_right_cfg(s):
    return dict(heads=s.heads, vdim=s.head_dim, state=s.state, groups=s.groups, conv=s.conv_taps, norm_groups=s.norm_groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", ["odd", "grouped", "large_state"])
def test_state_space_mixer_alone_in_portions(dtype, variant):
    """Portions of 1, 2, 7 and 40 tokens carry filter and state on; sizes: a state size that is no multiple of 4,
    norm parts that cut through heads, groups, more columns than a block's slice, a state of 130."""
    spec = {"odd": _ssd_spec(),
            "grouped": _ssd_spec(heads=4, head_dim=40, state=16, groups=2, conv_taps=2, norm_groups=1),
            "large_state": _ssd_spec(heads=2, head_dim=8, state=130, groups=2, conv_taps=3, norm_groups=2)}[variant]
    rt = _rt(dtype)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "R."), 11, 0.2, dtype=DT[dtype], device="cuda")
    w["R.A_log"] = torch.linspace(-2.0, 0.5, spec.heads, device="cuda").to(DT[dtype])     # slow and fast decays
    part = cls(spec, w, "R.", rt)
    cache = SequenceCache({0: cls.cache_need(spec)}, 64 * 4, DT[dtype], "cuda:0", max_seqs=3)
    cache.alloc_slot()
    slot = cache.alloc_slot()
    T = 700                                   # (portions of more than 128 tokens run in chunks side by side)
    x = (torch.randn(T, spec.hidden, generator=torch.Generator().manual_seed(4)) * 1.2).to(DT[dtype])
    ref = plain.right_mixer(x.double(), _w64(w), "R.", _plain_right_cfg(spec), spec.norm_eps)
    outs = []
    for lo, hi in _cuts(T, [1, 2, 1, 7, 40, 1, 129, 1, 300, 2, 128, 1]):
        ctx = _ctx([slot], [lo], [hi - lo])
        outs.append(part.forward(x[lo:hi].contiguous().cuda(), ctx, None, cache.state_of(0), True).sum(0))
    assert helpers.rel_err(torch.cat(outs), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parallel_mixer_is_the_weighted_sum_of_its_branches(dtype):
    left, right = _sink_spec(), _ssd_spec()
    spec = ParallelMixerSpec(hidden=40, prefix="mix.", branches=(MixerBranch(left, "left.", 0.8), MixerBranch(right, "right.", 1.7)))
    rt = _rt(dtype)
    cls = MIXERS.get(spec.kind)
    w = random_weights(cls.declare(spec, "l0."), 13, 0.25, dtype=DT[dtype], device="cuda")
    part = cls(spec, w, "l0.", rt)
    need = cls.cache_need(spec)
    assert need.kind == "full" and need.state_shape == (2 * (6 + 2) * 24 + 2 * 2 * 40 + 3 * (72 + 40) + 3 * 20 * 24,)
    cache = SequenceCache({0: need}, 64 * 4, DT[dtype], "cuda:0", max_seqs=2)
    slot = cache.alloc_slot()
    T = 70
    x = (torch.randn(T, 40, generator=torch.Generator().manual_seed(8)) * 1.2).to(DT[dtype])
    w64 = _w64(w)
    ref = (0.8 * plain.left_mixer(x.double(), w64, "l0.mix.left.", _plain_left_cfg(left))
           + 1.7 * plain.right_mixer(x.double(), w64, "l0.mix.right.", _plain_right_cfg(right), 1e-5))
    outs = []
    for lo, hi in _cuts(T, [33, 1, 1, 2, 30, 1]):
        cache.reserve([(slot, hi)]); cache.flush()
        ctx = _ctx([slot], [lo], [hi - lo])
        outs.append(part.forward(x[lo:hi].contiguous().cuda(), ctx, cache.view(0), cache.state_of(0), True).sum(0))
        cache.set_length(slot, hi)
    assert helpers.rel_err(torch.cat(outs), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_behind_and_in_front_in_one_pass(dtype):
    K = _rt(dtype).kernels
    g = torch.Generator().manual_seed(2)
    h0, y = torch.randn(7, 100, generator=g), torch.randn(7, 100, generator=g) * 3
    wp, wn = torch.rand(100, generator=g) + 0.5, torch.rand(100, generator=g) + 0.5
    want_h = h0.double() + plain.rms_norm(y.double(), wp.double(), 1e-3)
    for mode in ("norm", "cast", "none"):
        h = h0.clone().cuda()
        x = K.post_pre_norm(h, y.cuda(), wp.cuda(), 1e-3, w_pre=wn.cuda() if mode == "norm" else None, eps_pre=1e-2,
                            cast=mode == "cast")
        assert (h.cpu().double() - want_h).abs().max() < 1e-5
        if mode == "none":
            assert x is None
        else:
            want_x = plain.rms_norm(want_h, wn.double(), 1e-2) if mode == "norm" else want_h
            assert x.dtype == DT[dtype] and helpers.rel_err(x, want_x) < (1e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [96, 1024])
def test_norm_behind_and_in_front_gives_a_row_the_same_bits_in_any_step(dtype, hidden):
    """Rows of up to 1024 elements take a block per row in small steps and a warp per row in large ones: the same
    bits for a row either way, and the plain implementation's values."""
    K = _rt(dtype).kernels
    g = torch.Generator().manual_seed(5)
    h0, y = torch.randn(90, hidden, generator=g), torch.randn(90, hidden, generator=g) * 2
    wp, wn = torch.rand(hidden, generator=g) + 0.5, torch.rand(hidden, generator=g) + 0.5
    outs = {}
    for rows in (90, 9):
        h = h0[:rows].clone().cuda()
        x = K.post_pre_norm(h, y[:rows].contiguous().cuda(), wp.cuda(), 1e-5, w_pre=wn.cuda(), eps_pre=1e-5)
        outs[rows] = (h.cpu(), x.float().cpu())
    assert torch.equal(outs[90][0][:9], outs[9][0]) and torch.equal(outs[90][1][:9], outs[9][1])
    want_h = h0.double() + plain.rms_norm(y.double(), wp.double(), 1e-5)
    assert (outs[90][0].double() - want_h).abs().max() < 1e-5
    assert helpers.rel_err(outs[90][1], plain.rms_norm(want_h, wn.double(), 1e-5)) < (1e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gelu_gate_in_the_product_and_alone(dtype):
    """The tanh form of gelu as the epilogue of the gate/up product (bfloat16) and as a kernel of its own."""
    from idempotent_llm_b200.config.specs import GatedMLPNames, GatedMLPSpec
    from idempotent_llm_b200.parts import FEED_FORWARDS
    rt = _rt(dtype)
    spec = GatedMLPSpec(hidden=72, intermediate=200, names=GatedMLPNames("g", "u", "d"), activation="gelu_tanh")
    cls = FEED_FORWARDS.get(spec.kind)
    w = random_weights(cls.declare(spec, "F."), 4, 0.2, dtype=DT[dtype], device="cuda")
    x = (torch.randn(150, 72, generator=torch.Generator().manual_seed(1)) * 2).to(DT[dtype])
    got = cls(spec, w, "F.", rt).forward(x.cuda(), None).sum(0)
    w64, x64 = _w64(w), x.double()
    want = (plain.gelu_tanh(x64 @ w64["F.g"].T) * (x64 @ w64["F.u"].T)) @ w64["F.d"].T
    assert helpers.rel_err(got, want) < TOL[dtype]


# ------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def lunulix_dirs(tmp_path_factory):
    made = {}

    def get(name, dtype="bfloat16", seed=1, sharp=1.0):
        key = (name, dtype, seed, sharp)
        if key not in made:
            d = str(tmp_path_factory.mktemp(f"lunulix-{name}-{dtype}-{seed}"))

            def edit(n, t):            # sharper attention: single far keys carry real weight
                return (t.float() * sharp).to(t.dtype) if (sharp != 1.0 and n.endswith(".left.q")) else t
            helpers.make_lunulix_dir(helpers.LUNULIX[name](), d, seed=seed, dtype=DT[dtype], edit=edit)
            made[key] = d
        return made[key]
    return get


def _plain_logits(model_dir, tokens):
    cfg, w = helpers.read_lunulix(model_dir)
    return plain.forward(cfg, w, tokens)


def _step_all(lm, slot, tokens, lo, hi):
    return lm.engine.step([(slot, tokens[lo:hi])], [list(range(hi - lo))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompt_and_every_layer_against_plain(lunulix_dirs, name, dtype):
    d = lunulix_dirs(name, dtype)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    cfg, w = helpers.read_lunulix(d)
    toks = helpers.rand_ids(77, cfg["vocab"], 5)
    want, layers = plain.forward(cfg, w, toks, return_layers=True)
    seen = []

    def recording(inner):
        def forward(h, *a, **k):
            out = inner(h, *a, **k)
            after = out[0].clone()
            if out[1] is not None:                   # the normed delta of the layer's last sublayer, handed on
                out[1].add_into(after, lm.model.rt.kernels)
            seen.append(after)
            return out
        return forward
    for b in lm.model.blocks:
        b.forward = recording(b.forward)
    s = lm.engine.open()
    got = _step_all(lm, s, toks, 0, len(toks))
    assert _close(got, want, dtype)
    for i, h in enumerate(seen):
        assert _close(h, layers[i], dtype), f"stream after layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "S"])
def test_token_by_token_from_the_first_token_equals_the_prompt(lunulix_dirs, name, dtype):
    d = lunulix_dirs(name, dtype)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    toks = helpers.rand_ids(70, lm.spec.vocab_size, 9)
    want = _plain_logits(d, toks)
    s = lm.engine.open()
    whole = _step_all(lm, s, toks, 0, len(toks))
    lm.engine.close(s)
    s = lm.engine.open()
    one = torch.cat([_step_all(lm, s, toks, i, i + 1) for i in range(len(toks))])
    assert _close(one, want, dtype) and _close(whole, want, dtype)
    assert helpers.rel_err(one, whole) < (1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [[2], [3, 2, 64, 1, 2], [63, 2, 1, 1, 64], [64, 65], [1, 128, 2]])
def test_portions_of_several_sizes(lunulix_dirs, dtype, sizes):
    d = lunulix_dirs("P", dtype, sharp=3.0)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    toks = helpers.rand_ids(40 if sizes == [2] else 200, lm.spec.vocab_size, 21)
    want = _plain_logits(d, toks)
    s = lm.engine.open()
    got = torch.cat([_step_all(lm, s, toks, lo, hi) for lo, hi in _cuts(len(toks), sizes)])
    assert _close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone_with_slots_and_pages_used_again(lunulix_dirs, dtype):
    """Three requests of unlike lengths start in one step and decode together, the short ones leaving early; then
    the slots and pages they gave back serve other requests, whose state must start from nothing."""
    d = lunulix_dirs("P", dtype, sharp=2.0)
    lm = api.load(d, dtype=dtype, max_tokens=64 * 6, max_seqs=3)
    V = lm.spec.vocab_size
    rounds = [[helpers.rand_ids(n, V, 30 + n) for n in (1, 67, 130)], [helpers.rand_ids(n, V, 50 + n) for n in (129, 3, 64)]]
    extra = [12, 5, 9]
    for reqs in rounds:
        full = [r + helpers.rand_ids(e, V, len(r)) for r, e in zip(reqs, extra)]
        want = [_plain_logits(d, f) for f in full]
        slots = [lm.engine.open() for _ in reqs]
        got = [[] for _ in reqs]
        lg = lm.engine.step([(s, r) for s, r in zip(slots, reqs)], [list(range(len(r))) for r in reqs])
        off = 0
        for i, r in enumerate(reqs):
            got[i].append(lg[off:off + len(r)]); off += len(r)
        for step in range(max(extra)):
            live = [i for i in range(len(reqs)) if step < extra[i]]
            lg = lm.engine.step([(slots[i], [full[i][len(reqs[i]) + step]]) for i in live])
            for row, i in enumerate(live):
                got[i].append(lg[row:row + 1])
            for i in range(len(reqs)):
                if step == extra[i] - 1:
                    lm.engine.close(slots[i])
        for i in range(len(reqs)):
            assert _close(torch.cat(got[i]), want[i], dtype), f"request {i}"
    assert lm.engine.cache.pages_held() == 0


def _far_key_model(tmp, dtype):
    """A one-layer model whose first attention head looks for ONE key: queries and keys of that head are a large
    multiple of the embedding's first coordinate, which only token 1 has (sign +) against all others (sign -);
    without filter or rotation in the way the score of the marked key stands out by e^(large)."""
    cfg = helpers.lunulix_config([helpers.lunulix_layer(heads=2, kv_heads=1, dim=8, vdim=8, scale=1.0, lconv=0, rot_dims=0,
                                                        r_heads=1, r_vdim=8, state=4, rconv=2, norm_groups=1, ff=None,
                                                        left_scale=1.0, right_scale=0.05)],
                                 vocab=16, width=16, emb_scale=1.0, side_dim=0)

    def edit(n, t):
        if n == "embed":
            t = t.float(); t[:, 0] = -1.0; t[1, 0] = 1.0; return t.to(DT[dtype])
        if n in ("l0.mix.left.q", "l0.mix.left.k"):
            t = torch.zeros_like(t.float()); t[0, 0] = -1.0 if n.endswith("q") else 1.0; return t.to(DT[dtype])
        if n == "l0.norm1":
            return torch.ones_like(t)
        if n == "l0.mix.left.sink":
            return torch.full_like(t, -30.0)
        return t
    return helpers.make_lunulix_dir(cfg, tmp, seed=3, dtype=DT[dtype], edit=edit)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("where", [0, 63, 64, 65, 127, 128, 300])
def test_one_far_key_among_hundreds_in_prompts_and_in_decoding(tmp_path, dtype, where):
    """The marked token sits at a page's first or last place, or far back; every later query finds it, in a
    prompt, across portions and when decoding alone.  Without the mark the logits differ, so a lost key shows."""
    d = _far_key_model(str(tmp_path), dtype)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    T = 330
    toks = [2 + (i % 13) for i in range(T)]
    toks[where] = 1
    want = _plain_logits(d, toks)
    lost = list(toks); lost[where] = 2
    assert helpers.rel_err(_plain_logits(d, lost)[-1:], want[-1:]) > 0.05        # the key matters to the last query
    s = lm.engine.open()
    portions = _cuts(T, [where + 1, 2, 250])[:3]               # up to the mark, two tokens, up to 250, the rest alone
    got = torch.cat([_step_all(lm, s, toks, lo, hi) for lo, hi in portions]
                    + [_step_all(lm, s, toks, i, i + 1) for i in range(portions[-1][1], T)])
    assert _close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(lunulix_dirs, dtype):
    """Sequences of one, two and three tokens (fewer than a filter's taps), alone and as a batch, after the slot
    held a longer request."""
    d = lunulix_dirs("P", dtype)
    lm = api.load(d, dtype=dtype, max_tokens=256, max_seqs=3)
    V = lm.spec.vocab_size
    s = lm.engine.open()
    lm.engine.step([(s, helpers.rand_ids(90, V, 1))])
    lm.engine.close(s)
    reqs = [helpers.rand_ids(n, V, 70 + n) for n in (1, 2, 3)]
    slots = [lm.engine.open() for _ in reqs]
    lg = lm.engine.step(list(zip(slots, reqs)), [list(range(len(r))) for r in reqs])
    off = 0
    for r in reqs:
        assert _close(lg[off:off + len(r)], _plain_logits(d, r), dtype)
        off += len(r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graph", [True, False])
def test_long_decoding_of_a_batch(lunulix_dirs, dtype, graph):
    """200 single-token steps of two sequences (captured graphs or not): state, filters and pages carry on."""
    d = lunulix_dirs("P", dtype)
    lm = api.load(d, dtype=dtype, max_tokens=1024, max_seqs=2, use_graph=graph)
    V = lm.spec.vocab_size
    full = [helpers.rand_ids(40 + 200, V, 3), helpers.rand_ids(3 + 200, V, 4)]
    starts = [40, 3]
    slots = [lm.engine.open(), lm.engine.open()]
    lm.engine.step([(s, f[:n]) for s, f, n in zip(slots, full, starts)])
    last = None
    for k in range(200):
        last = lm.engine.step([(s, [f[n + k]]) for s, f, n in zip(slots, full, starts)])
    for row, f in enumerate(full):
        assert _close(last[row:row + 1], _plain_logits(d, f)[-1:], dtype)


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_drawn_configurations_in_a_batch_and_decoding(tmp_path, seed):
    """Configurations drawn at random (sizes, head counts, filters, rotations, state sizes, layer make-up): a prompt of
    200 tokens beside a short one, then six single tokens each, in both types."""
    cfg = helpers.lunulix_random_config(seed)
    d = helpers.make_lunulix_dir(cfg, str(tmp_path), seed=seed, std=0.08)
    V = cfg["vocab"]
    a, b = helpers.rand_ids(206, V, seed), helpers.rand_ids(9, V, seed + 100)
    want_a, want_b = _plain_logits(d, a), _plain_logits(d, b)
    for dtype in ("float32", "bfloat16"):
        lm = api.load(d, dtype=dtype, max_tokens=512)
        sa, sb = lm.engine.open(), lm.engine.open()
        g = lm.engine.step([(sa, a[:200]), (sb, b[:3])], [list(range(200)), [0, 1, 2]])
        ga, gb = [g[:200]], [g[200:]]
        for k in range(6):
            g = lm.engine.step([(sa, [a[200 + k]]), (sb, [b[3 + k]])])
            ga.append(g[0:1]); gb.append(g[1:2])
        assert _close(torch.cat(ga), want_a, dtype) and _close(torch.cat(gb), want_b, dtype), f"{dtype}: {cfg}"
        del lm


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(lunulix_dirs, dtype):
    """``LM.generate`` (scheduler, batching, sampling) against greedy decoding with the plain implementation."""
    d = lunulix_dirs("Q", dtype)
    lm = api.load(d, dtype=dtype, max_tokens=256)
    V = lm.spec.vocab_size
    prompts = [helpers.rand_ids(n, V, 80 + n) for n in (5, 1, 19)]
    toks, _ = lm.generate(prompts, max_new=6)
    cfg, w = helpers.read_lunulix(d)
    for p, row in zip(prompts, toks.tolist()):
        seq = list(p)
        for t in row:
            lg = plain.forward(cfg, w, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > (1e-3 if dtype == "float32" else 0.1):      # a near tie may fall either way
                assert t == int(lg.argmax())
            seq.append(t)


def test_the_command_line_replays_a_trace(lunulix_dirs, tmp_path):
    """``bin/trace_run`` on a Lunulix folder: whole, decoded and batched give the plain implementation's logits."""
    import json
    import subprocess
    import sys
    import numpy as np
    d = lunulix_dirs("P", "float32")
    V = helpers.LUNULIX["P"]()["vocab"]
    a, b = helpers.rand_ids(70, V, 1), helpers.rand_ids(9, V, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for k in range(4):
        steps.append({"step": k + 1, "entries": [{"id": "a", "tokens": [a[66 + k]], "want": [0]}, {"id": "b", "tokens": [b[5 + k]], "want": [0] if k == 3 else []}],
                      "end": ["a", "b"] if k == 3 else []})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]})
    p = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                        "--out", str(tmp_path), "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(6)]
    read = lambda i: torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{i}.f32"), dtype="<f4").reshape(-1, V).copy())
    wa, wb = _plain_logits(d, a), _plain_logits(d, b)
    assert helpers.rel_err(read(0), torch.stack([wa[0], wa[65], wb[4]])) < TOL["float32"]
    assert helpers.rel_err(read(4), torch.stack([wa[69], wb[8]])) < TOL["float32"]
    assert helpers.rel_err(read(5), wb[8:9]) < TOL["float32"]
    assert helpers.rel_err(read(5), read(4)[1:2]) < 1e-5
