"""Lusalorn through the engine against the plain NumPy statement of the design (plain_lusalorn.py):
each mechanism alone, whole prompts, token-by-token decoding, prompts in portions, unequal batches,
slots and pages used again, keys at page borders and at the windows' edges, long decoding, odd sizes,
and greedy generation through the library's own entry point."""
import functools
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_lusalorn as plain
import helpers
from helpers import run_batch, run_tail_one_by_one, run_whole
from math_utils_b200 import DecoderModel, LLM, StepEntry
from math_utils_b200.weights.safetensors import write_safetensors

pytestmark = pytest.mark.gpu

# Every sublayer's output is brought to unit rms before it joins the stream, so a sublayer's rounding noise enters
# the stream at full size however small the sublayer's output was: the rows' noise is larger than in a design that
# norms inputs.  (A key that is wrongly seen or missed moves a row by tens of percent.)
# Configuration b joins every sublayer at the stream's own size (multiplier 1) at a width of 50: more noise still.
BF16_RMS = {"a": 0.02, "b": 0.05, "c": 0.02}


def check_logits(got, want, dtype, what=""):
    helpers.check_logits(got, want, dtype, what, bf16_rms=BF16_RMS[what.split()[1]])

YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


def attention(heads, kv_heads, dim, vdim, window, scale, rot_dims, base=10000.0, diff=0.25, scaling=None, kv_from=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = scaling
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale,
         "diff": diff, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def parallel(left, right, left_scale, right_scale):
    heads, kv_heads, dim, vdim, scale, rot_dims, base, scaling = left
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = scaling
    s_heads, s_vdim, state, groups, conv, norm_groups = right
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot},
        "right": {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups},
        "left_scale": left_scale, "right_scale": right_scale}}


def with_mlp(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


def config(vocab, width, mult, eps, big, layers):
    return {"architecture": "Lusalorn", "vocab": vocab, "width": width, "residual_mult": mult, "norm": {"eps": eps},
            "embedding": {"bigram": {"buckets": big[0], "mul_prev": big[1], "mul_cur": big[2]}}, "layers": layers}


# a window shorter than a page; a borrowing layer with a WIDER window than its owner's; a layer without feed-forward
_A = attention(4, 2, 16, 24, 40, 0.25, 8)
CFG_A = config(300, 64, 0.5, 1e-6, (97, 7, 3), [
    with_mlp(_A, 96),
    with_mlp(parallel((4, 1, 16, 8, 0.25, 16, 5.0e4, YARN), (4, 8, 16, 2, 4, 1), 0.7, 1.3), 96),
    with_mlp(attention(4, 2, 16, 24, 70, 0.25, 8, kv_from=0, diff=0.1), 80),
    with_mlp(parallel((2, 2, 8, 16, 0.35, 4, 100.0, None), (2, 16, 8, 1, 2, 2), 1.0, 0.5), None)])
# nothing a multiple of 8; a window of one (a token sees itself only) and one longer than any prompt here; as many
# kv heads as heads; one group; two taps; rotation over fewer entries than a map has; stretched rotation in the
# windowed layer; a large eps
CFG_B = config(131, 50, 1.0, 1e-3, (11, 1000003, 1), [
    with_mlp(parallel((2, 1, 10, 7, 0.3, 6, 300.0, None), (3, 5, 7, 1, 2, 3), 0.4, 1.7), 33),
    with_mlp(attention(3, 3, 6, 5, 1, 0.4, 4, base=50.0), 21),
    with_mlp(attention(3, 1, 6, 9, 1000, 0.4, 6, base=50.0, diff=0.6, scaling=YARN), 21)])
# sizes the tensor-core kernels take; the state-space layer first; a borrowing layer; windows that end inside a page
_C = attention(4, 2, 32, 64, 100, 0.18, 16, base=5.0e5, scaling={"factor": 5.0, "original": 128, "fast": 20.0, "slow": 1.5})
CFG_C = config(384, 128, 0.35, 2e-5, (251, 29, 13), [
    with_mlp(parallel((4, 2, 64, 32, 0.125, 64, 1.0e6, YARN), (4, 32, 64, 2, 4, 2), 0.65, 1.15), 256),
    with_mlp(_C, 256),
    with_mlp(dict(_C, mixer=dict(_C["mixer"], kv_from=1, mask={"size": 64})), 256),
    with_mlp(parallel((8, 2, 32, 32, 0.18, 32, 1.0e4, None), (8, 16, 32, 4, 3, 1), 1.0, 1.0), 128)])
CONFIGS = {"a": CFG_A, "b": CFG_B, "c": CFG_C}


@functools.lru_cache(maxsize=None)
def weights_of(name):
    return plain.random_weights(CONFIGS[name], seed=sum(map(ord, name)) + 23)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        d = str(tmp_path_factory.mktemp(f"lusalorn_{name}"))
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        write_safetensors(os.path.join(d, "model.safetensors"),
                          {k: torch.from_numpy(np.array(v)).to(torch.bfloat16) for k, v in weights_of(name).items()})
        out[name] = d
    return out


_models = {}


def engine(folders, name, dtype):
    key = (name, dtype)
    if key not in _models:
        model = DecoderModel.from_dir(folders[name], dtype=dtype)
        _models[key] = (model, model.new_cache(max_tokens=64 * 24, n_slots=8))
    return _models[key]


def tokens_for(name, n, seed=0):
    return np.random.default_rng(2000 + seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


_plain_cache = {}


def plain_logits(name, tokens):
    key = (name, tuple(tokens))
    if key not in _plain_cache:
        _plain_cache[key] = plain.forward(CONFIGS[name], weights_of(name), list(tokens))
    return _plain_cache[key]


CASES = [(n, d) for n in CONFIGS for d in ("float32", "bfloat16")]


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompt_and_every_layer(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 150)
    layers = []
    want = plain.forward(CONFIGS[name], weights_of(name), toks, layers)
    slot = cache.acquire()
    trace = {}
    got = model.step(cache, [StepEntry(slot, toks, list(range(len(toks))))], trace=trace).cpu().numpy()
    cache.release(slot)
    if dtype == "float32":
        for i, x in enumerate(layers):
            assert np.abs(trace[f"h.{i}.res2"] - x).max() < 1e-4, f"residual stream after layer {i}"
    check_logits(got, want, dtype, f"lusalorn {name} whole prompt")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_then_token_by_token(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 150, seed=1)                 # the tail crosses the page border at 128 and every window's edge
    got = run_tail_one_by_one(model, cache, toks, tail=120)
    check_logits(got, plain_logits(name, toks), dtype, f"lusalorn {name} tail one by one")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("portions", [(2, 3, 59, 1, 64, 21), (64, 64, 22), (127, 2, 2, 19), (1, 1, 1, 147), (2,) * 12 + (126,)])
def test_prompt_in_portions(folders, name, dtype, portions):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, sum(portions), seed=2)
    slot = cache.acquire()
    rows, at = [], 0
    for n in portions:
        rows.append(model.step(cache, [StepEntry(slot, toks[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    cache.release(slot)
    check_logits(np.concatenate(rows), plain_logits(name, toks), dtype, f"lusalorn {name} portions {portions}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batch_against_each_alone(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    lens, prompts = (140, 5, 66, 131), (129, 1, 33, 64)
    requests = [tokens_for(name, n, seed=10 + i) for i, n in enumerate(lens)]
    got = run_batch(model, cache, requests, prompts)
    for i, r in enumerate(requests):
        check_logits(got[i], plain_logits(name, r), dtype, f"lusalorn {name} batch request {i}")
        if dtype == "float32":
            alone = run_tail_one_by_one(model, cache, r, tail=lens[i] - prompts[i])
            assert np.abs(alone - got[i]).max() < 2e-5, "a request's logits depend on its batch"


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "bfloat16"), ("c", "float32")])
def test_slots_pages_and_state_used_again(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    free = [cache.free_pages(g.index) for g in cache.kv_groups]
    first = tokens_for(name, 200, seed=20)
    second = tokens_for(name, 90, seed=21)
    a = run_whole(model, cache, first)
    slot = cache.acquire()                               # the slot, the pages and the state the first request held
    model.step(cache, [StepEntry(slot, second[:70], [])])
    b = [model.step(cache, [StepEntry(slot, [t], [0])]).cpu().numpy() for t in second[70:]]
    cache.release(slot)
    assert [cache.free_pages(g.index) for g in cache.kv_groups] == free
    check_logits(a, plain_logits(name, first), dtype, f"lusalorn {name} first holder")
    check_logits(np.concatenate(b), plain_logits(name, second)[70:], dtype, f"lusalorn {name} second holder of the same slot")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "bfloat16")])
@pytest.mark.parametrize("n", [1, 2, 3, 39, 40, 41, 63, 64, 65, 70, 71, 99, 100, 101, 128, 129, 193])
def test_lengths_around_page_borders_and_window_edges(folders, name, dtype, n):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 193, seed=30)[:n]
    slot = cache.acquire()
    got = model.step(cache, [StepEntry(slot, toks, [0, n - 1])]).cpu().numpy()
    cache.release(slot)
    want = plain_logits(name, tokens_for(name, 193, seed=30))          # causal: a prefix's logits are the long prompt's
    check_logits(got, want[[0, n - 1]], dtype, f"lusalorn {name} prompt of {n}")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "bfloat16")])
def test_long_decoding(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 270, seed=40)
    free = [cache.free_pages(g.index) for g in cache.kv_groups]
    got = run_tail_one_by_one(model, cache, toks, tail=267)            # three tokens, then one by one over four pages
    check_logits(got, plain_logits(name, toks), dtype, f"lusalorn {name} long decoding")
    assert [cache.free_pages(g.index) for g in cache.kv_groups] == free


def test_windowed_cache_gives_pages_back(folders):
    model, cache = engine(folders, "c", "float32")
    windowed = [g for g in cache.kv_groups if g.spec.window > 0]
    assert windowed and windowed[0].spec.window == 100
    slot = cache.acquire()
    model.step(cache, [StepEntry(slot, tokens_for("c", 400, seed=41), [])])
    assert windowed[0].pages_held(slot) <= 3                            # 100 positions lie in three pages at most
    cache.release(slot)


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_greedy_generation_through_the_library(folders, name):
    llm = LLM(folders[name], dtype="float32", temperature=0.0, max_tokens=24, context=512)
    assert llm.model.graph_safe                                            # single-token steps replay from a graph
    prompts = [tokens_for(name, n, seed=50 + n) for n in (70, 3, 129)]
    outs = llm.generate(prompts)
    for p, out in zip(prompts, outs):
        assert len(out) == 24
        seq = list(p)
        for tok in out:
            row = plain.forward(CONFIGS[name], weights_of(name), seq)[-1]
            best = int(np.argmax(row))
            assert tok == best or row[best] - row[tok] < 1e-4, f"greedy token {len(seq) - len(p)} of a prompt of {len(p)}"
            seq.append(tok)
    alone = llm.generate([prompts[2]])[0]
    assert alone == outs[2], "a request generates other tokens alone than in a batch"
    from math_utils_b200 import SamplingParams
    from math_utils_b200.engine.generate import generate
    eager = generate(llm.model, [prompts[0]], 24, SamplingParams(0.0, 1, 0), context=512, use_graph=False)[0]
    assert eager == outs[0], "eager steps and replayed steps generate different tokens"


def test_requests_that_end_early_leave_the_others_alone(folders):
    """A stop token ends some requests early: the batch thins out, the rest moves to a smaller recorded step (whose
    set-up run must not move recurrent state or the last token on), and nobody's tokens change."""
    llm = LLM(folders["a"], dtype="float32", temperature=0.0, max_tokens=30, context=512)
    prompts = [tokens_for("a", n, seed=70 + n) for n in (40, 9, 66, 3, 21)]
    free = llm.generate(prompts, stop_ids=[])
    # a token that request 0 produces early and request 2 later, if there is one; else request 0's sixth token
    stop = free[0][5]
    want = []
    for out in free:
        want.append(out[:out.index(stop)] if stop in out else out)
    assert len(want[0]) <= 5 and any(len(w) == 30 for w in want), "the test's premise: some end early, some run on"
    got = llm.generate(prompts, stop_ids=[stop])
    assert got == want
    assert llm.generate(prompts[1:], stop_ids=[stop]) == want[1:]


def test_conversation_on_a_kept_slot(folders):
    """Two turns through ``LLM.prompt``: the slot keeps keys, values, the recurrence's state and the last token."""
    llm = LLM(folders["a"], dtype="float32", temperature=0.0, max_tokens=9, context=512)
    first, second = tokens_for("a", 45, seed=60), tokens_for("a", 30, seed=61)
    out1 = llm.prompt(first)
    out2 = llm.prompt(second)
    seq = list(first) + out1 + list(second)
    assert len(out1) == 9 and len(out2) == 9
    for tok in out2:
        row = plain.forward(CONFIGS["a"], weights_of("a"), seq)[-1]
        best = int(np.argmax(row))
        assert tok == best or row[best] - row[tok] < 1e-4
        seq.append(tok)


# ------------------------------------------------------------------ mechanisms alone
def _ops():
    from math_utils_b200.csrc import ops
    return ops


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device="cuda", dtype=dtype)


def ints(a):
    return dev(np.asarray(a), torch.int32)


def test_token_pair_embedding_kernel():
    ops, rng = _ops(), np.random.default_rng(1)
    V, D, buckets, mp, mc = 50, 20, 13, 1000003, 7
    w = {"embed": rng.normal(0, 1, (V, D)), "bigram": rng.normal(0, 1, (buckets + 1, D))}
    big = {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}
    seqs = [rng.integers(0, V, n).tolist() for n in (5, 1, 9)]
    last = torch.full((6,), -7, dtype=torch.int32, device="cuda")
    slots = [4, 0, 2]
    # first portions: 3, 1 and 4 tokens; then the rest of the first and third (the second has ended); then single tokens
    steps = [[(0, 0, 3), (1, 0, 1), (2, 0, 4)], [(0, 3, 4), (2, 4, 6)], [(0, 4, 5), (2, 6, 7)], [(2, 7, 8)], [(2, 8, 9)]]
    for step in steps:
        ids = np.concatenate([seqs[s][a:b] for s, a, b in step])
        pos = np.concatenate([np.arange(a, b) for s, a, b in step])
        seq = np.concatenate([[i] * (b - a) for i, (s, a, b) in enumerate(step)])
        first = np.cumsum([0] + [b - a for s, a, b in step])
        single = all(b - a == 1 for s, a, b in step)
        got = ops.embed_pair(ints(ids), ints(pos), ints(seq), ints(first), ints([slots[s] for s, a, b in step]), last,
                             dev(w["embed"]), dev(w["bigram"]), mp, mc, single).cpu().numpy()
        want = np.concatenate([plain.embedding(seqs[s], w, big)[a:b] for s, a, b in step])
        assert np.abs(got - want).max() < 1e-6, f"step {step}"
        for s, a, b in step:
            assert int(last[slots[s]]) == seqs[s][b - 1]
    assert int(last[1]) == -7                                           # slots of no sequence are left alone


def test_output_norm_kernel():
    ops, rng = _ops(), np.random.default_rng(2)
    x, w = rng.normal(0, 3, (9, 44)), rng.normal(0, 0.2, 44)
    for eps in (1e-6, 0.5):                               # an eps that matters: inside the root, not outside
        want = plain.output_norm(x, {"n": w}, "n", eps)
        assert np.abs(ops.rms_norm_out(dev(x), dev(w), eps, offset=1.0).cpu().numpy() - want).max() < 3e-6
        rows = ints([5, 0, 8])
        assert np.abs(ops.rms_norm_out(dev(x), dev(w), eps, offset=1.0, rows=rows).cpu().numpy() - want[[5, 0, 8]]).max() < 3e-6
        stream = rng.normal(0, 1, (9, 44))
        acc, copy = dev(stream), torch.zeros((9, 44), dtype=torch.bfloat16, device="cuda")
        ops.rms_norm_out(dev(x), dev(w), eps, offset=1.0, scale=0.35, out=acc, add=True, copy=copy)
        assert np.abs(acc.cpu().numpy() - (stream + 0.35 * want)).max() < 3e-6
        assert (copy == acc.to(torch.bfloat16)).all()
        # two branches that join with a weight each, summed by the same launch
        x2 = rng.normal(0, 2, (9, 44))
        acc = dev(stream)
        ops.rms_norm_out(dev(x), dev(w), eps, offset=1.0, scale=0.35, out=acc, add=True, second=(0.7, dev(x2), 1.2))
        want2 = plain.output_norm(0.7 * x + 1.2 * x2, {"n": w}, "n", eps)
        assert np.abs(acc.cpu().numpy() - (stream + 0.35 * want2)).max() < 3e-6
    # rows that are no whole 16-byte pieces, and rows longer than a block keeps in registers
    for n in (45, 5000):
        x, w = rng.normal(0, 3, (3, n)), rng.normal(0, 0.2, n)
        want = plain.output_norm(x, {"n": w}, "n", 1e-5)
        assert np.abs(ops.rms_norm_out(dev(x), dev(w), 1e-5, offset=1.0).cpu().numpy() - want).max() < 5e-6


def test_gated_activation_and_weighted_sum_kernels():
    ops, rng = _ops(), np.random.default_rng(3)
    a = rng.normal(0, 2, (7, 2 * 19))
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 3e-2)):
        ad = dev(a, dtype)
        out = torch.zeros((7, 19), device="cuda", dtype=dtype)
        ops.gated_act(ad, out, "silu")
        af = ad.float().cpu().numpy().astype(np.float64)
        assert np.abs(out.float().cpu().numpy() - plain.silu(af[:, :19]) * af[:, 19:]).max() < tol
    p, q, y = rng.normal(0, 1, (5, 11)), rng.normal(0, 1, (5, 11)), rng.normal(0, 1, (5, 11))
    yd = dev(y)
    ops.scaled_sum(dev(p), 0.7, dev(q), 1.2, yd)
    assert np.abs(yd.cpu().numpy() - (0.7 * p + 1.2 * q)).max() < 1e-6
    ops.scaled_sum(dev(p), 0.7, dev(q), 1.2, yd, add=True)
    assert np.abs(yd.cpu().numpy() - 2 * (0.7 * p + 1.2 * q)).max() < 1e-6


def _paged(rng, lens, width, page=64):
    """Rows of several sequences in pages handed out in a scrambled order."""
    n_pages = sum(-(-n // page) for n in lens) + 3
    order = rng.permutation(n_pages)
    pages = np.zeros((n_pages, page, width))
    table = np.zeros((len(lens), 24), dtype=np.int32)
    seqs, at = [], 0
    for s, n in enumerate(lens):
        rows = rng.normal(0, 1, (n, width))
        seqs.append(rows)
        for i in range(-(-n // page)):
            table[s, i] = order[at]
            chunk = rows[i * page:(i + 1) * page]
            pages[order[at], :len(chunk)] = chunk
            at += 1
    return seqs, pages, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,maps,dim,vdim,rot_dims", [(4, 2, 2, 16, 24, 8), (3, 3, 1, 6, 5, 4), (2, 1, 2, 10, 7, 10),
                                                                  (4, 1, 1, 64, 32, 0)])
def test_query_key_preparation_kernel(dtype, heads, kv_heads, maps, dim, vdim, rot_dims):
    ops, rng = _ops(), np.random.default_rng(4)
    from math_utils_b200.parts.position import rotary_frequencies
    eps = 1e-2
    rot = {"base": 300.0, "dims": rot_dims, "scaling": YARN}
    positions = np.array([0, 63, 64, 130, 5, 40000])
    seq_of = np.array([0, 0, 1, 1, 2, 2])
    table = np.zeros((3, 700), dtype=np.int32)
    table[0, :2], table[1, :3], table[2, 0], table[2, 625] = (4, 1), (2, 6, 5), 3, 0
    T, qw, kw, vw = len(positions), heads * maps * dim, kv_heads * maps * dim, kv_heads * vdim
    proj = dev(rng.normal(0, 2, (T, qw + kw + vw)), dtype)
    x = proj.float().cpu().numpy().astype(np.float64)
    wq, wk = rng.normal(1, 0.2, dim), rng.normal(1, 0.2, dim)
    want_q = plain.normed_rotated(x[:, :qw].reshape(T, heads, maps, dim), wq, positions, rot, eps).reshape(T, qw)
    want_k = plain.normed_rotated(x[:, qw:qw + kw].reshape(T, kv_heads, maps, dim), wk, positions, rot, eps).reshape(T, kw)
    rows = torch.zeros((7, 64, kw + vw), device="cuda", dtype=dtype)
    freqs, mag = rotary_frequencies(rot_dims, rot["base"], rot["scaling"])
    pf, pm = plain.rotary_frequencies(rot)
    assert np.allclose(freqs, pf, rtol=1e-12) and abs(mag - pm) < 1e-12
    q = proj[:, :qw]
    ops.qk_prepare(q, proj[:, qw:qw + kw], proj[:, qw + kw:], dev(wq), dev(wk), dev(np.array(freqs or [0.0])), mag, rot_dims,
                   eps, heads, kv_heads, maps, dim, vdim, ints(positions), ints(seq_of), ints(table), 64, rows)
    tol = (1e-5 + 40000 * 2.0 ** -23 * 3) if dtype == torch.float32 else 4e-2      # float32 angles at position 40,000
    assert np.abs(q.float().cpu().numpy() - want_q).max() < tol
    got = rows.float().cpu().numpy()
    for t, (p, s) in enumerate(zip(positions, seq_of)):
        row = got[table[s, p // 64], p % 64]
        assert np.abs(row[:kw] - want_k[t]).max() < tol
        assert np.abs(row[kw:] - x[t, qw + kw:]).max() == 0.0
    assert np.count_nonzero(got.reshape(-1, kw + vw).any(axis=1)) == T       # no other row was touched
    # queries alone, for a layer that reads another layer's rows
    proj2 = dev(x, dtype)
    ops.qk_prepare(proj2[:, :qw], None, None, dev(wq), None, dev(np.array(freqs or [0.0])), mag, rot_dims, eps, heads,
                   kv_heads, maps, dim, vdim, ints(positions), None, None, 64, None)
    assert np.abs(proj2[:, :qw].float().cpu().numpy() - want_q).max() < tol


def _plain_mapped(q, rows, pos, maps, dim, vdim, H, G, scale, window, lam, out_scale, eps):
    """One token's heads [H, vdim] from its sequence's rows, through the plain functions."""
    n = pos + 1
    k = rows[:n, :G * maps * dim].reshape(n, G, maps, dim)
    v = rows[:n, G * maps * dim:].reshape(n, G, vdim)
    qq = np.zeros((n, H, maps, dim))
    qq[-1] = q.reshape(H, maps, dim)
    a = [plain.softmax_attention(qq[:, :, m], k[:, :, m], v, scale, window)[-1] for m in range(maps)]
    if maps == 1:
        return a[0] * out_scale
    return plain.unit_rms(a[0] - lam * a[1], eps) * out_scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,maps,dim,vdim,window", [(4, 2, 2, 16, 24, 40), (3, 3, 1, 6, 5, 1), (2, 1, 2, 10, 7, 0),
                                                      (4, 2, 1, 64, 32, 100), (8, 2, 2, 32, 64, 64), (2, 2, 2, 8, 200, 129)])
def test_mapped_attention_kernel(dtype, H, G, maps, dim, vdim, window):
    ops, rng = _ops(), np.random.default_rng(5)
    lens = [1, 2, 63, 64, 65, 300, 1400]
    width = G * (maps * dim + vdim)
    seqs, pages, table = _paged(rng, lens, width)
    scale, lam, out_scale, eps = 0.37, 0.45, 0.8, 1e-3
    if dtype == torch.bfloat16:                                       # the cache holds what bfloat16 can hold
        pages = dev(pages, dtype).float().cpu().numpy().astype(np.float64)
        seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
    # queries: the last position of every sequence, and some in the middle of the longest
    picks = [(s, n - 1) for s, n in enumerate(lens)] + [(5, p) for p in (0, 63, 64, 127, 128, 191, 192, 250, 251)] + [(6, 1100)]
    q = rng.normal(0, 1, (len(picks), H, maps, dim)) / math.sqrt(dim) * 3
    # Keys that stand out.  For the query at 299 of the long sequence: head 0's first map points at the oldest key
    # it sees (or a far one without a window), so that key's value must come through; the last head's first map
    # points at the key just OUTSIDE the window, which must change nothing.
    w_eff = window if window else 300
    inside, outside = max(0, 299 - w_eff + 1), 299 - w_eff
    key_of = lambda j, g, m: seqs[5][j, (g * maps + m) * dim:(g * maps + m + 1) * dim]
    q[5, 0, 0] = key_of(inside, 0, 0) * 30.0 / scale / (key_of(inside, 0, 0) ** 2).sum()
    if outside >= 0:
        g_last = (H - 1) // (H // G)
        q[5, H - 1, 0] = key_of(outside, g_last, 0) * 30.0 / scale / (key_of(outside, g_last, 0) ** 2).sum()
    if dtype == torch.bfloat16:
        q = dev(q, dtype).float().cpu().numpy().astype(np.float64)
    want = np.stack([_plain_mapped(q[i], seqs[s], p, maps, dim, vdim, H, G, scale, window, lam, out_scale, eps)
                     for i, (s, p) in enumerate(picks)])
    if maps == 1 and window != 1:
        v_inside = seqs[5][inside, G * maps * dim: G * maps * dim + vdim]
        assert np.abs(want[5, 0] / out_scale - v_inside).max() < 0.3 * np.abs(v_inside).max()      # the test's own premise
    out = torch.zeros((len(picks), H * vdim), device="cuda", dtype=dtype)
    ops.mapped_attention(dev(q.reshape(len(picks), -1), dtype), dev(pages, dtype), ints(table), 64,
                         ints([p for _, p in picks]), ints([s for s, _ in picks]), H, G, maps, dim, vdim, scale, window, out,
                         lam=lam, out_scale=out_scale, eps=eps, unit_rms=maps == 2)
    got = out.float().cpu().numpy().reshape(len(picks), H, vdim)
    err = np.abs(got - want).max(axis=(1, 2))
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    assert err.max() < tol, f"first wrong query {int(np.argmax(err > tol))}: {picks[int(np.argmax(err > tol))]}"
    # the same queries through the kernel of single-token steps (pages shared out over blocks, then merged)
    out.zero_()
    ops.mapped_attention(dev(q.reshape(len(picks), -1), dtype), dev(pages, dtype), ints(table), 64,
                         ints([p for _, p in picks]), ints([s for s, _ in picks]), H, G, maps, dim, vdim, scale, window, out,
                         lam=lam, out_scale=out_scale, eps=eps, unit_rms=maps == 2, single_tokens=True)
    got = out.float().cpu().numpy().reshape(len(picks), H, vdim)
    err = np.abs(got - want).max(axis=(1, 2))
    assert err.max() < tol, f"single tokens: first wrong query {int(np.argmax(err > tol))}: {picks[int(np.argmax(err > tol))]}"


@pytest.mark.parametrize("H,G,maps,dim,vdim,window", [(4, 2, 2, 16, 16, 40), (2, 1, 2, 64, 128, 100), (8, 2, 1, 128, 64, 0),
                                                      (3, 3, 1, 32, 48, 1), (4, 4, 2, 80, 112, 64), (2, 2, 2, 32, 32, 129)])
def test_mapped_attention_on_tensor_cores_prompt_tiles(H, G, maps, dim, vdim, window):
    """Several sequences' tokens in one step as tiles of up to 64, each token with its own causal edge and window;
    some sequences bring only their last tokens (the rows before them are in the cache already)."""
    ops, rng = _ops(), np.random.default_rng(8)
    lens, new = [130, 1, 64, 65, 7, 200], [130, 1, 64, 3, 7, 70]           # cached lengths, and how many of them are this step's
    width = G * (maps * dim + vdim)
    seqs, pages, table = _paged(rng, lens, width)
    scale, lam, out_scale, eps = 0.21, 0.45, 0.8, 1e-3
    pages = dev(pages, torch.bfloat16).float().cpu().numpy().astype(np.float64)
    seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
    tok_seq = np.repeat(np.arange(len(lens)), new)
    tok_pos = np.concatenate([np.arange(n - k, n) for n, k in zip(lens, new)])
    T = len(tok_seq)
    q = rng.normal(0, 1, (T, H, maps, dim)) / math.sqrt(dim) * 4
    # the last token of the longest sequence: one head points at the oldest key it sees, another at the key just outside
    w_eff = window if window else 200
    inside, outside = max(0, 199 - w_eff + 1), 199 - w_eff
    key_of = lambda j, g: seqs[5][j, g * maps * dim:g * maps * dim + dim]
    q[T - 1, 0, 0] = key_of(inside, 0) * 30.0 / scale / (key_of(inside, 0) ** 2).sum()
    if outside >= 0:
        g_last = (H - 1) // (H // G)
        q[T - 1, H - 1, 0] = key_of(outside, g_last) * 30.0 / scale / (key_of(outside, g_last) ** 2).sum()
    q = dev(q, torch.bfloat16).float().cpu().numpy().astype(np.float64)
    tiles, at = [], 0
    for k in new:
        tiles += [(at + o, min(64, k - o)) for o in range(0, k, 64)]
        at += k
    tiles.sort(key=lambda t: -tok_pos[t[0] + t[1] - 1])
    want = np.stack([_plain_mapped(q[t], seqs[tok_seq[t]], tok_pos[t], maps, dim, vdim, H, G, scale, window, lam, out_scale, eps)
                     for t in range(T)])
    outs = []
    for tc in (True, False):
        out = torch.zeros((T, H * vdim), device="cuda", dtype=torch.bfloat16)
        before = ops.launch_count
        ops.mapped_attention(dev(q.reshape(T, -1), torch.bfloat16), dev(pages, torch.bfloat16), ints(table), 64, ints(tok_pos),
                             ints(tok_seq), H, G, maps, dim, vdim, scale, window, out, lam=lam, out_scale=out_scale, eps=eps,
                             unit_rms=maps == 2, tiles=ints(np.array(tiles)), tensor_cores=tc)
        got = out.float().cpu().numpy().reshape(T, H, vdim)
        err = np.abs(got - want).max(axis=(1, 2))
        bad = int(np.argmax(err > 4e-2))
        assert err.max() < 4e-2, f"tensor cores {tc}: first wrong token {bad} (sequence {tok_seq[bad]}, position {tok_pos[bad]})"
        outs.append(got)
    assert np.abs(outs[0] - outs[1]).max() < 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,P,N,groups,taps,parts", [(4, 8, 16, 2, 4, 1), (3, 5, 7, 1, 2, 3), (4, 32, 64, 2, 4, 2),
                                                         (2, 64, 128, 1, 3, 1), (6, 16, 8, 3, 1, 2), (2, 12, 200, 1, 2, 1)])
def test_state_space_kernels(dtype, heads, P, N, groups, taps, parts):
    """Convolution, recurrence and gated norm against the plain mixer with identity matrices around them, a prompt
    cut into steps of several sizes for two sequences that share the steps."""
    ops, rng = _ops(), np.random.default_rng(6)
    inner, ch = heads * P, heads * P + 2 * groups * N
    wide = 2 * inner + 2 * groups * N + heads
    m = {"heads": heads, "vdim": P, "state": N, "groups": groups, "conv": taps, "norm_groups": parts}
    eps = 1e-3
    w = {"in": np.eye(wide), "o": np.eye(inner), "conv": rng.normal(0, 0.5, (ch, taps)), "conv.b": rng.normal(0, 0.1, ch),
         "dt_bias": rng.uniform(-3, 0.5, heads), "A_log": rng.uniform(-1, 1.5, heads), "D": rng.normal(1, 0.3, heads),
         "norm": rng.normal(1, 0.2, inner)}
    lens = [37, 21]
    us = [dev(rng.normal(0, 1, (n, wide)), dtype) for n in lens]
    want = [plain.state_space(u.float().cpu().numpy().astype(np.float64), m, w, "", eps) for u in us]
    state = torch.full((5, (taps - 1) * ch + heads * N * P), 9.0, device="cuda")
    slots = [3, 1]
    state[slots] = 0.0                                                   # what taking a slot does
    cuts = [[(0, 2), (2, 3), (3, 20), (20, 21), (21, 22), (22, 37)], [(0, 1), (1, 3), (3, 20), (20, 21), (21, 21), (21, 21)]]
    got = [[], []]
    for step in range(6):
        live = [s for s in range(2) if cuts[s][step][1] > cuts[s][step][0]]
        u = torch.cat([us[s][cuts[s][step][0]:cuts[s][step][1]] for s in live])
        counts = [cuts[s][step][1] - cuts[s][step][0] for s in live]
        T = sum(counts)
        seq = ints(np.repeat(np.arange(len(live)), counts))
        first, sl = ints(np.cumsum([0] + counts)), ints([slots[s] for s in live])
        xbc = torch.zeros((T, ch), device="cuda")
        ops.ssd_conv(u[:, inner:inner + ch], dev(w["conv"]), dev(w["conv.b"]), seq, first, sl, state, all(c == 1 for c in counts), xbc)
        y = torch.zeros((T, inner), device="cuda")
        ops.ssd_scan(xbc, u[:, inner + ch:], dev(w["dt_bias"]), dev(w["A_log"]), dev(w["D"]), heads, P, N, groups, first, sl,
                     state, (taps - 1) * ch, y)
        out = torch.zeros((T, inner), device="cuda", dtype=dtype)
        ops.gated_group_norm(y, u[:, :inner], dev(w["norm"]), parts, eps, out)
        at = 0
        for s, c in zip(live, counts):
            got[s].append(out[at:at + c].float().cpu().numpy())
            at += c
    for s in range(2):
        err = np.abs(np.concatenate(got[s]) - want[s]).max(axis=1)
        tol = 5e-5 if dtype == torch.float32 else 4e-2
        assert err.max() < tol * max(1.0, np.abs(want[s]).max()), f"sequence {s}: first wrong token {int(np.argmax(err > tol))}"
    assert (state[[0, 2, 4]] == 9.0).all()                              # other slots' state is left alone
