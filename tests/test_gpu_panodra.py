"""The Panodra decoder on the GPU against the plain implementation (``plain_panodra.py``): every mechanism alone,
then whole models through the engine: prompts, token-by-token decoding, portions, unequal batches, slots and pages
used again, far keys at page and run borders, first tokens, long decoding, greedy generation, and the trace replay
program."""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_panodra as plain
from idempotent_llm_b200 import api
from idempotent_llm_b200.cache import SequenceCache
from idempotent_llm_b200.config import (DenseMLPSpec, DyTNormSpec, LatentAttentionSpec, RampScaling, RotarySpec,
                                        TableExpertsSpec)
from idempotent_llm_b200.engine.batch import context_from_packed, pack_step_host
from idempotent_llm_b200.parts import FEED_FORWARDS, MIXERS, NORMS, Runtime
from idempotent_llm_b200.weights import random_weights

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# against the 64-bit plain implementation, relative to the largest value: 32-bit arithmetic rounds at 6e-8 a few
# hundred times per layer; bfloat16 rounds activations at 4e-3 a handful of times per layer.  A wrong mechanism
# shows at 1e-2 and above.
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
F64 = torch.float64


def _close(got, want, dtype):
    """32-bit: the largest difference relative to the largest value.  bfloat16: the root mean square of the difference
    relative to that of the values, and a looser bound on the largest one."""
    if dtype == "float32":
        return helpers.rel_err(got, want) < TOL[dtype]
    g, w = got.detach().double().cpu(), want.detach().double().cpu()
    rms = float((g - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt())
    return rms < TOL[dtype] and helpers.rel_err(got, want) < 0.25


def _rt(dtype):
    from idempotent_llm_b200.kernels import Kernels
    dev = torch.device("cuda:0")
    return Runtime(device=dev, dtype=DT[dtype], kernels=Kernels(DT[dtype], dev))


def _ctx(slots, starts, lens, tokens=None):
    toks = tokens if tokens is not None else [[0] * L for L in lens]
    packed, n, q_lens = pack_step_host(slots, starts, toks)
    return context_from_packed(packed.cuda(), n, slots, q_lens, starts, host_tokens=tokens)


def _w64(w):
    return {k: (v.double().cpu() if v.is_floating_point() else v.cpu()) for k, v in w.items()}


def _cuts(T, sizes):
    out, lo, i = [], 0, 0
    while lo < T:
        n = sizes[min(i, len(sizes) - 1)]
        out.append((lo, min(T, lo + n)))
        lo, i = lo + n, i + 1
    return out


# ----------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,width", [(3, 20), (200, 64), (5, 1030)])
def test_norm_without_statistics_adds_and_norms_and_picks_rows(dtype, n, width):
    rt = _rt(dtype)
    spec = DyTNormSpec(size=width, weight="n")
    cls = NORMS.get("dyt")
    w = random_weights(cls.declare(spec, "L."), 3, 0.3, dtype=DT[dtype], device="cuda")
    norm = cls(spec, w, "L.", rt)
    g = torch.Generator().manual_seed(n)
    h, delta = torch.randn(n, width, generator=g) * 2, torch.randn(1, n, width, generator=g)
    w64 = _w64(w)
    want = plain.dyt(h.double() + delta[0].double(), w64["L.n.alpha"], w64["L.n"], w64["L.n.b"])
    hd = h.cuda()
    got = norm.forward(hd, delta.cuda(), None)
    assert helpers.rel_err(got, want) < (1e-6 if dtype == "float32" else 8e-3)
    assert torch.equal(hd.cpu(), h + delta[0])                                  # the stream took the delta, in 32-bit
    rows = torch.tensor([n - 1, 0], dtype=torch.int32, device="cuda")
    before = hd.clone()
    picked = norm.forward(hd, None, None, rows=rows)
    assert torch.equal(picked, got[[n - 1, 0]]) and torch.equal(hd, before)


def _latent_spec(**kw):
    base = dict(hidden=40, n_heads=3, plain_dim=12, rot_dim=8, value_dim=20, kv_rank=24, softmax_scale=0.3, eps=1e-5,
                position=RotarySpec(3e4, 8, 1 << 20, variant="interleaved", scaling=RampScaling(4.0, 64.0, 8.0, 1.0)), sink=True)
    base.update(kw)
    return LatentAttentionSpec(**base)


def _plain_mixer_cfg(s):
    rot = dict(base=s.position.theta, dims=s.position.dim)
    if s.position.scaling is not None:
        sc = s.position.scaling
        rot["scaling"] = dict(factor=sc.factor, original=sc.original, fast=sc.fast, slow=sc.slow)
    return dict(heads=s.n_heads, dim=s.plain_dim, rot_dim=s.rot_dim, vdim=s.value_dim, kv_rank=s.kv_rank, scale=s.softmax_scale, rot=rot)


LATENT_SHAPES = {
    "all": _latent_spec(),
    "no sink, no scaling": _latent_spec(sink=False, position=RotarySpec(1e4, 8, 1 << 20, variant="interleaved")),
    "one head, odd sizes": _latent_spec(hidden=20, n_heads=1, plain_dim=6, rot_dim=6, value_dim=10, kv_rank=13,
                                        position=RotarySpec(5e5, 6, 1 << 20, variant="interleaved")),
    "more heads than a block has warps": _latent_spec(hidden=48, n_heads=11, plain_dim=8, rot_dim=4, value_dim=8, kv_rank=16,
                                                      position=RotarySpec(1e4, 4, 1 << 20, variant="interleaved")),
    "twenty heads on fragments": _latent_spec(hidden=64, n_heads=20, plain_dim=16, rot_dim=16, value_dim=24, kv_rank=32,
                                              position=RotarySpec(1e4, 16, 1 << 20, variant="interleaved"), softmax_scale=0.2),
    "tensor-core head 64": _latent_spec(hidden=64, n_heads=4, plain_dim=32, rot_dim=32, value_dim=48, kv_rank=64,
                                        position=RotarySpec(1e4, 32, 1 << 20, variant="interleaved"), softmax_scale=0.12),
    "tensor-core head 128, wide latent": _latent_spec(hidden=64, n_heads=2, plain_dim=64, rot_dim=16, value_dim=128, kv_rank=288,
                                                      position=RotarySpec(1e4, 16, 1 << 20, variant="interleaved",
                                                                          scaling=RampScaling(2.0, 32.0, 4.0, 1.0)), softmax_scale=0.1),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", sorted(LATENT_SHAPES))
def test_latent_attention_alone_in_prompts_portions_and_single_tokens(dtype, shape):
    """Two sequences side by side: the whole prompt in one step; then the same tokens in portions (64 + 3 + 200 + 1 ...)
    and the rest one by one, so that whole prompts (the tensor-core kernel where it fits), portions behind a prefix
    (one run), and single tokens (runs of 256 keys that meet in scratch) are all compared with the plain mixer."""
    s = LATENT_SHAPES[shape]
    rt = _rt(dtype)
    cls = MIXERS.get("latent_attention")
    w = random_weights(cls.declare(s, "M."), 7, 0.25, dtype=DT[dtype], device="cuda")
    mixer = cls(s, w, "M.", rt)
    T = [300, 70]
    g = torch.Generator().manual_seed(11)
    x = [(torch.randn(t, s.hidden, generator=g)).to(DT[dtype]) for t in T]
    w64 = _w64(w)
    want = [plain.latent_attention(xi.double(), _plain_mixer_cfg(s), w64, "M.", s.eps) for xi in x]
    need = cls.cache_need(s)
    for sizes in ([400], [64, 3, 200, 1]):
        cache = SequenceCache({0: need}, 1024, DT[dtype], "cuda", max_seqs=4)
        slots = [cache.alloc_slot(), cache.alloc_slot()]
        got = [[], []]
        at = 0
        while at < max(T):
            n = sizes.pop(0) if sizes else 1
            live = [i for i in range(2) if at < T[i]]
            lens = [min(n, T[i] - at) for i in live]
            cache.reserve([(slots[i], at + L) for i, L in zip(live, lens)])
            cache.flush()
            ctx = _ctx([slots[i] for i in live], [at] * len(live), lens)
            xs = torch.cat([x[i][at:at + L] for i, L in zip(live, lens)]).cuda()
            y = mixer.forward(xs, ctx, cache.view(0), None, True).sum(0)
            off = 0
            for i, L in zip(live, lens):
                got[i].append(y[off:off + L].cpu()); off += L
                cache.set_length(slots[i], at + L)
            at += n
        for i in range(2):
            assert _close(torch.cat(got[i]), want[i], dtype), f"sequence {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sink", [-30.0, 0.0, 6.0])
def test_a_sink_far_below_at_and_above_the_scores(dtype, sink):
    s = _latent_spec()
    rt = _rt(dtype)
    cls = MIXERS.get("latent_attention")
    w = random_weights(cls.declare(s, "M."), 9, 0.25, dtype=DT[dtype], device="cuda")
    w["M.sink"] = torch.full_like(w["M.sink"], sink)
    mixer = cls(s, w, "M.", rt)
    x = torch.randn(40, s.hidden, generator=torch.Generator().manual_seed(1)).to(DT[dtype])
    want = plain.latent_attention(x.double(), _plain_mixer_cfg(s), _w64(w), "M.", s.eps)
    if sink == 6.0:     # the sink matters: without it the first token's output is hundreds of times larger
        none = {k: v for k, v in _w64(w).items() if k != "M.sink"}
        assert plain.latent_attention(x.double(), _plain_mixer_cfg(s), none, "M.", s.eps)[0].abs().max() > 50 * want[0].abs().max()
    cache = SequenceCache({0: cls.cache_need(s)}, 256, DT[dtype], "cuda", max_seqs=2)
    slot = cache.alloc_slot()
    cache.reserve([(slot, 40)]); cache.flush()
    whole = mixer.forward(x.cuda(), _ctx([slot], [0], [40]), cache.view(0), None, True).sum(0)
    last = mixer.forward(x[39:].cuda(), _ctx([slot], [39], [1]), cache.view(0), None, True).sum(0)      # the same token again, alone
    assert _close(whole, want, dtype) and _close(last, want[39:], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_dense_feed_forward_with_the_square_of_relu(dtype):
    rt = _rt(dtype)
    for hidden, inter, n in ((72, 200, 150), (20, 28, 5)):
        spec = DenseMLPSpec(hidden=hidden, intermediate=inter)
        cls = FEED_FORWARDS.get(spec.kind)
        w = random_weights(cls.declare(spec, "F."), 4, 0.2, dtype=DT[dtype], device="cuda")
        x = (torch.randn(n, hidden, generator=torch.Generator().manual_seed(1)) * 2).to(DT[dtype])
        part = cls(spec, w, "F.", rt)
        want = plain.dense_ff(x.double(), _w64(w), "F.")
        assert helpers.rel_err(part.forward(x.cuda(), None).sum(0), want) < TOL[dtype]
        h = torch.ones(n, hidden, device="cuda")
        out = part.forward(x.cuda(), None, residual=h)
        got = h - 1.0 if out is None else out.sum(0)
        assert helpers.rel_err(got, want) < TOL[dtype] * 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,inter,experts,top,n", [(64, 48, 5, 3, 7), (64, 48, 5, 3, 300), (20, 12, 3, 2, 40), (32, 16, 1, 1, 200),
                                                        (128, 96, 9, 2, 1000)])
def test_table_experts_few_tokens_and_grouped_by_expert(dtype, hidden, inter, experts, top, n):
    """Steps of few tokens look the experts up on the device (token by token, expert by expert, or every expert over
    all tokens, by the step's size); steps of many tokens whose ids the host holds run grouped by expert; all against
    the plain sum.  An expert no token of the step uses has no rows."""
    rt = _rt(dtype)
    V = 23
    spec = TableExpertsSpec(hidden=hidden, intermediate=inter, n_experts=experts, top=top, vocab_size=V)
    cls = FEED_FORWARDS.get(spec.kind)
    w = random_weights(cls.declare(spec, "F."), 6, 0.2, dtype=DT[dtype], device="cuda")
    part = cls(spec, w, "F.", rt)
    toks = helpers.rand_ids(n, V if n < 1000 else 2, n)               # (the largest step uses two token ids only)
    x = torch.randn(n, hidden, generator=torch.Generator().manual_seed(2)).to(DT[dtype])
    want = plain.table_experts(x.double(), toks, dict(router=dict(top=top)), _w64(w), "F.")
    for host in (True, False):
        ctx = _ctx([0, 1], [0, 0], [n - n // 3, n // 3], tokens=[toks[:n - n // 3], toks[n - n // 3:]])
        if not host:
            ctx.host_tokens = None
        h = torch.full((n, hidden), 0.5, device="cuda")
        assert part.forward(x.cuda(), ctx, residual=h) is None
        assert helpers.rel_err(h - 0.5, want) < TOL[dtype] * 2, f"host tokens {host}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logits_times_a_constant_then_capped(dtype):
    K = _rt(dtype).kernels
    l = torch.linspace(-200, 200, 1001)
    got = K.logit_cap(l.clone().cuda().reshape(7, 143), 0.7, 22.0).cpu().reshape(-1)
    assert (got.double() - 22.0 * torch.tanh(l.double() * 0.7 / 22.0)).abs().max() < 1e-5 and float(got.abs().max()) < 22.0
    assert torch.equal(K.logit_cap(l.clone().cuda(), 2.0, 0.0).cpu(), l * 2.0)


# ------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def panodra_dirs(tmp_path_factory):
    made = {}

    def get(name, dtype="bfloat16", seed=1, sharp=1.0):
        key = (name, dtype, seed, sharp)
        if key not in made:
            d = str(tmp_path_factory.mktemp(f"panodra-{name}-{dtype}-{seed}"))

            def edit(n, t):            # sharper attention: single far keys carry real weight
                return (t.float() * sharp).to(t.dtype) if (sharp != 1.0 and n.endswith(".mix.q")) else t
            # (the widest model with the default spread of weights lets its stream grow to ~150, where rounding
            # flips saturated norms: narrower weights keep it a test of the mechanisms)
            helpers.make_panodra_dir(helpers.PANODRA[name](), d, seed=seed, dtype=DT[dtype], edit=edit,
                                     std=0.08 if name == "T" else 0.2)
            made[key] = d
        return made[key]
    return get


def _plain_logits(model_dir, tokens):
    cfg, w = helpers.read_model_dir(model_dir)
    return plain.forward(cfg, w, tokens)


def _step_all(lm, slot, tokens, lo, hi):
    return lm.engine.step([(slot, tokens[lo:hi])], [list(range(hi - lo))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "T"])
def test_whole_prompt_and_every_layer_run_against_plain(panodra_dirs, name, dtype):
    d = panodra_dirs(name, dtype)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    cfg, w = helpers.read_model_dir(d)
    toks = helpers.rand_ids(150, cfg["vocab"], 5)
    layers = []
    want = plain.forward(cfg, w, toks, layers)
    seen = []

    def recording(inner):
        def forward(h, *a, **k):
            out = inner(h, *a, **k)
            seen.append(out[0].clone() if out[1] is None else out[0] + out[1].sum(0))
            return out
        return forward
    for b in lm.model.blocks:
        b.forward = recording(b.forward)
    s = lm.engine.open()
    got = _step_all(lm, s, toks, 0, len(toks))
    assert len(seen) == len(layers)                      # a layer of the loop counts every time it runs
    for i, h in enumerate(seen):
        assert _close(h, layers[i], dtype), f"stream after layer run {i}"
    assert _close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "T"])
def test_token_by_token_from_the_first_token_equals_the_prompt(panodra_dirs, name, dtype):
    d = panodra_dirs(name, dtype)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    toks = helpers.rand_ids(70, lm.spec.vocab_size, 9)
    want = _plain_logits(d, toks)
    s = lm.engine.open()
    whole = _step_all(lm, s, toks, 0, len(toks))
    lm.engine.close(s)
    s = lm.engine.open()
    one = torch.cat([_step_all(lm, s, toks, i, i + 1) for i in range(len(toks))])
    assert _close(one, want, dtype) and _close(whole, want, dtype)
    assert helpers.rel_err(one, whole) < (1e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [[2], [3, 2, 64, 1, 2], [63, 2, 1, 1, 64], [64, 65], [1, 128, 2], [2, 320, 3]])
def test_portions_of_several_sizes(panodra_dirs, dtype, sizes):
    d = panodra_dirs("A", dtype, sharp=2.0)
    lm = api.load(d, dtype=dtype, max_tokens=512)
    toks = helpers.rand_ids(40 if sizes == [2] else 340 if sizes[1:2] == [320] else 200, lm.spec.vocab_size, 21)
    want = _plain_logits(d, toks)
    s = lm.engine.open()
    got = torch.cat([_step_all(lm, s, toks, lo, hi) for lo, hi in _cuts(len(toks), sizes)])
    assert _close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "T"])
def test_unequal_batch_against_each_alone_with_slots_and_pages_used_again(panodra_dirs, name, dtype):
    """Three requests of unlike lengths start in one step and decode together, the short ones leaving early; then the
    slots and pages they gave back serve other requests."""
    d = panodra_dirs(name, dtype, sharp=2.0)
    lm = api.load(d, dtype=dtype, max_tokens=64 * 6, max_seqs=3)
    V = lm.spec.vocab_size
    waves = [[helpers.rand_ids(n, V, 30 + n) for n in (1, 67, 130)], [helpers.rand_ids(n, V, 50 + n) for n in (129, 3, 64)]]
    extra = [12, 5, 9]
    for reqs in waves:
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_through_layers_of_growing_head_counts(tmp_path, dtype):
    """1 200 tokens (the tensor-core kernel shares a long tile's runs among several blocks and spreads them over a pool
    by head group) through a layer of 2 heads followed by layers of 8 and 5: what one layer's plan holds must not
    serve another's head count.  Then 20 single tokens beside a second, shorter sequence."""
    cfg = helpers.panodra_config([
        helpers.panodra_layer(heads=2, dim=32, rot_dim=32, vdim=48, kv_rank=64, scale=0.12, ff=96),
        helpers.panodra_layer(sink=True, heads=8, dim=16, rot_dim=16, vdim=16, kv_rank=32, scale=0.18, mlp="moe", ff=32, experts=3, top=2),
        helpers.panodra_layer(heads=5, dim=48, rot_dim=16, vdim=72, kv_rank=96, scale=0.12, mlp=None)],
        vocab=300, width=128, loop=(0, 2, 2), logit_scale=1.0, softcap=20.0)
    d = helpers.make_panodra_dir(cfg, str(tmp_path), seed=7, dtype=DT[dtype], std=0.08)
    T, V = 1220, 300
    a, b = helpers.rand_ids(T, V, 3), helpers.rand_ids(150, V, 4)
    want_a, want_b = _plain_logits(d, a), _plain_logits(d, b)
    lm = api.load(d, dtype=dtype, max_tokens=2048)
    sa, sb = lm.engine.open(), lm.engine.open()
    places = list(range(0, T - 20, 13))
    g = lm.engine.step([(sa, a[:T - 20]), (sb, b[:130])], [places, [129]])
    assert _close(g[:len(places)], want_a[places], dtype) and _close(g[len(places):], want_b[129:130], dtype)
    rows_a, rows_b = [], []
    for k in range(20):
        g = lm.engine.step([(sa, [a[T - 20 + k]]), (sb, [b[130 + k]])])
        rows_a.append(g[0:1]); rows_b.append(g[1:2])
    assert _close(torch.cat(rows_a), want_a[T - 20:], dtype) and _close(torch.cat(rows_b), want_b[130:], dtype)


def _far_key_model(tmp, dtype, sink):
    """A one-layer model whose first head looks for ONE key.  The embedding's first coordinate is -1 for every token but
    token 1 (+1); the latent's first number reads it (the other rows of the down projection are zero, so the normed
    latent is (+-sqrt(rank), 0, ...)), the head's first unrotated key dim copies it, and its query is a large negative
    multiple of the same coordinate: the marked key's score stands out by e^(large), no rotation in the way."""
    cfg = helpers.panodra_config([helpers.panodra_layer(sink=sink, heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, scale=1.0, mlp=None)],
                                 vocab=16, width=16, loop=None, logit_scale=1.0, softcap=None)

    def edit(n, t):
        f = t.float()
        if n == "embed":
            f[:, 0] = -1.0; f[1, 0] = 1.0
        elif n == "l0.mix.q":
            f = torch.zeros_like(f); f[0, 0] = -8.0
        elif n == "l0.mix.dkv":
            f = torch.zeros_like(f); f[0, 0] = 1.0
        elif n == "l0.mix.uk":
            f = torch.zeros_like(f); f[0, 0] = 1.0
        elif n in ("l0.norm1", "l0.mix.dkv.norm"):
            f = torch.ones_like(f)
        elif n == "l0.norm1.b":
            f = torch.zeros_like(f)
        elif n == "l0.norm1.alpha":
            f = torch.ones_like(f)
        elif n == "l0.mix.sink":
            f = torch.full_like(f, 2.0)
        return f.to(t.dtype)
    return helpers.make_panodra_dir(cfg, tmp, seed=3, dtype=DT[dtype], std=0.3, edit=edit)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("where", [0, 63, 64, 65, 255, 256, 257, 300])
def test_one_far_key_among_hundreds_in_prompts_and_in_decoding(tmp_path, dtype, where):
    """The marked token sits at a page's or a run's first or last place, or far back; every later query finds it, in a
    prompt, across portions and when decoding alone.  Without the mark the logits differ, so a lost key shows."""
    d = _far_key_model(str(tmp_path), dtype, sink=where % 2 == 0)
    lm = api.load(d, dtype=dtype, max_tokens=1024)
    T = 330
    toks = [2 + (i % 13) for i in range(T)]
    toks[where] = 1
    want = _plain_logits(d, toks)
    lost = list(toks); lost[where] = 2
    assert helpers.rel_err(_plain_logits(d, lost)[-1:], want[-1:]) > 0.05        # the key matters to the last query
    s = lm.engine.open()
    whole = _step_all(lm, s, toks, 0, T)
    lm.engine.close(s)
    s = lm.engine.open()
    portions = _cuts(T, [where + 1, 2, 250])[:3]               # up to the mark, two tokens, up to 250, the rest alone
    got = torch.cat([_step_all(lm, s, toks, lo, hi) for lo, hi in portions]
                    + [_step_all(lm, s, toks, i, i + 1) for i in range(portions[-1][1], T)])
    assert _close(got, want, dtype) and _close(whole, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(panodra_dirs, dtype):
    """Sequences of one, two and three tokens, alone and as a batch, after the slot held a longer request."""
    d = panodra_dirs("A", dtype)
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
def test_long_decoding_of_a_batch(panodra_dirs, dtype, graph):
    """300 single-token steps of two sequences (captured graphs or not), across page borders and the border of a run
    of keys."""
    d = panodra_dirs("A", dtype)
    lm = api.load(d, dtype=dtype, max_tokens=1024, max_seqs=2, use_graph=graph)
    V = lm.spec.vocab_size
    full = [helpers.rand_ids(40 + 300, V, 3), helpers.rand_ids(3 + 300, V, 4)]
    starts = [40, 3]
    slots = [lm.engine.open(), lm.engine.open()]
    lm.engine.step([(s, f[:n]) for s, f, n in zip(slots, full, starts)])
    last = None
    for k in range(300):
        last = lm.engine.step([(s, [f[n + k]]) for s, f, n in zip(slots, full, starts)])
    for row, f in enumerate(full):
        assert _close(last[row:row + 1], _plain_logits(d, f)[-1:], dtype)


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_drawn_configurations_in_a_batch_and_decoding(tmp_path, seed):
    """Configurations drawn at random (sizes, head counts, sinks, scaled rotations, feed-forwards, loops, constants): a
    prompt of 200 tokens beside a short one, then six single tokens each, in both types."""
    cfg = helpers.panodra_random_config(seed)
    d = helpers.make_panodra_dir(cfg, str(tmp_path), seed=seed, std=0.08)
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
def test_greedy_generation_through_the_entry_point(panodra_dirs, dtype):
    """``LM.generate`` (scheduler, batching, sampling) against greedy decoding with the plain implementation."""
    d = panodra_dirs("C", dtype)
    lm = api.load(d, dtype=dtype, max_tokens=256)
    V = lm.spec.vocab_size
    prompts = [helpers.rand_ids(n, V, 80 + n) for n in (5, 1, 19)]
    toks, _ = lm.generate(prompts, max_new=6)
    cfg, w = helpers.read_model_dir(d)
    for p, row in zip(prompts, toks.tolist()):
        seq = list(p)
        for t in row:
            lg = plain.forward(cfg, w, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > (1e-3 if dtype == "float32" else 0.1):      # a near tie may fall either way
                assert t == int(lg.argmax())
            seq.append(t)


def test_the_command_line_replays_a_trace(panodra_dirs, tmp_path):
    """``bin/trace_run`` on a Panodra folder: whole, decoded and batched give the plain implementation's logits."""
    d = panodra_dirs("A", "float32")
    V = helpers.PANODRA["A"]()["vocab"]
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
