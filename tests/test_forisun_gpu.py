"""Forisun through the engine against the plain NumPy statement of the design (plain_forisun.py):
each kernel alone, whole prompts, token-by-token decoding, prompts in portions, unequal batches,
slots and pages used again, page borders, long decoding, odd sizes, and greedy generation through
the library's own entry point."""
import functools
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_forisun as plain
from helpers import check_logits, run_batch, run_tail_one_by_one, run_whole
from math_utils_b200 import DecoderModel, LLM, StepEntry
from math_utils_b200.weights.safetensors import write_safetensors

pytestmark = pytest.mark.gpu


def mixer(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, dims=None, scaling=None, kv_from=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling:
        rot["scaling"] = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(experts, top, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def layer(m, mlp):
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}
# moe first, a dense layer in the middle, two layers that borrow caches, one without a feed-forward
_A = mixer(3, 16, 8, 24, 32, 0.2, scaling=YARN)
CFG_A = {"architecture": "Forisun", "vocab": 300, "width": 64, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
         "layers": [layer(_A, moe(6, 2, 48, 1.5)), layer(_A, {"kind": "dense", "ff": 96}),
                    layer(dict(_A, kv_from=0), moe(6, 2, 48, 1.5)), layer(dict(_A, kv_from=1), None)]}
# nothing a multiple of 8; one head; all experts chosen; one expert chosen; fewer rotated entries than the
# rotated part holds; no stretching; layers of different sizes (two cache groups)
_B1 = mixer(5, 4, 6, 3, 20, 0.31, base=500.0)
CFG_B = {"architecture": "Forisun", "vocab": 131, "width": 50, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-3},
         "layers": [layer(mixer(1, 10, 6, 7, 12, 0.4, base=100.0, dims=4), {"kind": "dense", "ff": 33}),
                    layer(_B1, moe(3, 3, 10, 0.9)),
                    layer(dict(_B1, heads=2, dim=9, vdim=11, kv_from=1), moe(5, 1, 14, 2.0))]}
# sizes the tensor-core products take
_C = mixer(4, 32, 16, 32, 64, 0.15, base=5.0e5, scaling={"factor": 5.0, "original": 128, "fast": 20.0, "slow": 1.5})
CFG_C = {"architecture": "Forisun", "vocab": 384, "width": 128, "embedding": {"scale": 1.0}, "norm": {"eps": 2e-5},
         "layers": [layer(_C, {"kind": "dense", "ff": 256}), layer(_C, moe(8, 2, 64, 1.8)),
                    layer(dict(_C, kv_from=1), moe(8, 2, 64, 1.8))]}
CONFIGS = {"a": CFG_A, "b": CFG_B, "c": CFG_C}


@functools.lru_cache(maxsize=None)
def weights_of(name, dtype="float32"):
    """Random weights.  The bfloat16 runs get routers that rounding cannot tip: a choice between two experts
    whose scores nearly tie is a matter of noise there, and one flipped choice moves a whole row of logits.
    Their routers barely depend on the token and the corrections lie 0.3 apart, so the choice is the same for
    every token; routing that varies from token to token is what the float32 runs and the kernel's own test
    (exact choices, bfloat16 rows) cover."""
    w = plain.random_weights(CONFIGS[name], seed=sum(map(ord, name)) + 11)
    if dtype == "bfloat16":
        rng = np.random.default_rng(5)
        for k in list(w):
            if k.endswith(".router"):
                w[k] = w[k] * np.float32(0.0625)
            if k.endswith(".correction"):
                w[k] = (rng.permutation(len(w[k])) * 0.3125).astype(np.float32)
    return w


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        for dtype in ("float32", "bfloat16"):
            d = str(tmp_path_factory.mktemp(f"forisun_{name}_{dtype}"))
            with open(os.path.join(d, "config.json"), "w") as f:
                json.dump(cfg, f)
            write_safetensors(os.path.join(d, "model.safetensors"),
                              {k: torch.from_numpy(np.array(v)).to(torch.bfloat16) for k, v in weights_of(name, dtype).items()})
            out[name, dtype] = d
    return out


_models = {}


def engine(folders, name, dtype):
    key = (name, dtype)
    if key not in _models:
        model = DecoderModel.from_dir(folders[name, dtype], dtype=dtype)
        _models[key] = (model, model.new_cache(max_tokens=64 * 24, n_slots=8))
    return _models[key]


def tokens_for(name, n, seed=0):
    return np.random.default_rng(1000 + seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


_plain_cache = {}


def plain_logits(name, tokens, dtype):
    key = (name, tuple(tokens), dtype)
    if key not in _plain_cache:
        _plain_cache[key] = plain.forward(CONFIGS[name], weights_of(name, dtype), list(tokens))
    return _plain_cache[key]


CASES = [(n, d) for n in CONFIGS for d in ("float32", "bfloat16")]


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompt_and_every_layer(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 150)
    layers = []
    want = plain.forward(CONFIGS[name], weights_of(name, dtype), toks, layers)
    slot = cache.acquire()
    trace = {}
    got = model.step(cache, [StepEntry(slot, toks, list(range(len(toks))))], trace=trace).cpu().numpy()
    cache.release(slot)
    if dtype == "float32":
        for i, x in enumerate(layers):
            assert np.abs(trace[f"h.{i}.res2"] - x).max() < 1e-4, f"residual stream after layer {i}"
    check_logits(got, want, dtype, f"forisun {name} whole prompt")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_then_token_by_token(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 150, seed=1)                 # the tail crosses the page border at 128
    got = run_tail_one_by_one(model, cache, toks, tail=45)
    check_logits(got, plain_logits(name, toks, dtype), dtype, f"forisun {name} tail one by one")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("portions", [(2, 3, 59, 1, 64, 21), (64, 64, 22), (127, 2, 2, 19), (1, 1, 1, 147)])
def test_prompt_in_portions(folders, name, dtype, portions):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, sum(portions), seed=2)
    slot = cache.acquire()
    rows, at = [], 0
    for n in portions:
        rows.append(model.step(cache, [StepEntry(slot, toks[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    cache.release(slot)
    check_logits(np.concatenate(rows), plain_logits(name, toks, dtype), dtype, f"forisun {name} portions {portions}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batch_against_each_alone(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    lens, prompts = (140, 5, 66, 131), (129, 1, 33, 64)
    requests = [tokens_for(name, n, seed=10 + i) for i, n in enumerate(lens)]
    got = run_batch(model, cache, requests, prompts)
    for i, r in enumerate(requests):
        check_logits(got[i], plain_logits(name, r, dtype), dtype, f"forisun {name} batch request {i}")
        if dtype == "float32":
            alone = run_tail_one_by_one(model, cache, r, tail=lens[i] - prompts[i])
            assert np.abs(alone - got[i]).max() < 2e-5, "a request's logits depend on its batch"


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "bfloat16")])
def test_slots_and_pages_used_again(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    free = [cache.free_pages(g.index) for g in cache.kv_groups]
    first = tokens_for(name, 200, seed=20)
    second = tokens_for(name, 90, seed=21)
    a = run_whole(model, cache, first)
    slot = cache.acquire()                               # the slot and the pages the first request held
    model.step(cache, [StepEntry(slot, second[:70], [])])
    b = [model.step(cache, [StepEntry(slot, [t], [0])]).cpu().numpy() for t in second[70:]]
    cache.release(slot)
    assert [cache.free_pages(g.index) for g in cache.kv_groups] == free
    check_logits(a, plain_logits(name, first, dtype), dtype, "first holder")
    check_logits(np.concatenate(b), plain_logits(name, second, dtype)[70:], dtype, "second holder of the same pages")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "bfloat16")])
@pytest.mark.parametrize("n", [1, 2, 63, 64, 65, 127, 128, 129, 192, 193])
def test_lengths_around_page_borders(folders, name, dtype, n):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 193, seed=30)[:n]
    slot = cache.acquire()
    got = model.step(cache, [StepEntry(slot, toks, [0, n - 1])]).cpu().numpy()
    cache.release(slot)
    want = plain_logits(name, tokens_for(name, 193, seed=30), dtype)          # causal: a prefix's logits are the long prompt's
    check_logits(got, want[[0, n - 1]], dtype, f"forisun {name} prompt of {n}")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("c", "bfloat16")])
def test_long_decoding(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 270, seed=40)
    got = run_tail_one_by_one(model, cache, toks, tail=267)            # three tokens, then one by one over four pages
    check_logits(got, plain_logits(name, toks, dtype), dtype, f"forisun {name} long decoding")


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_through_the_library(folders, name):
    llm = LLM(folders[name, "float32"], dtype="float32", temperature=0.0, max_tokens=24, context=512)
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


# ------------------------------------------------------------------ mechanisms alone
def _ops():
    from math_utils_b200.csrc import ops
    return ops


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device="cuda", dtype=dtype)


def test_dynamic_tanh_kernel():
    ops, rng = _ops(), np.random.default_rng(1)
    x, w, b, alpha = rng.normal(0, 2, (37, 50)), rng.normal(1, 0.3, 50), rng.normal(0, 0.3, 50), 0.63
    want = plain.dynamic_tanh(x, w, b, alpha)
    args = (dev(x), dev(w), dev(b), dev(np.array([alpha])))
    assert np.abs(ops.dynamic_tanh(*args).cpu().numpy() - want).max() < 2e-6
    assert np.abs(ops.dynamic_tanh(*args, out_dtype=torch.bfloat16).float().cpu().numpy() - want).max() < 2e-2
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device="cuda")
    assert np.abs(ops.dynamic_tanh(*args, rows=rows).cpu().numpy() - want[[5, 0, 36]]).max() < 2e-6
    acc = dev(rng.normal(0, 1, (37, 50)))
    before = acc.cpu().numpy().copy()
    ops.dynamic_tanh(*args, out=acc, add=True)
    assert np.abs(acc.cpu().numpy() - (before + want)).max() < 2e-6


def test_rms_norm_kernel():
    ops, rng = _ops(), np.random.default_rng(2)
    x, w = rng.normal(0, 3, (9, 44)), rng.normal(1, 0.2, 44)
    for eps in (1e-6, 0.5):                               # an eps that matters: inside the root, not outside
        want = plain.rms_norm(x, w, eps)
        assert np.abs(ops.rms_norm(dev(x), dev(w), eps).cpu().numpy() - want).max() < 3e-6


@pytest.mark.parametrize("scaling", [None, YARN, {"factor": 6.0, "original": 1024, "fast": 24.0, "slow": 2.0}])
@pytest.mark.parametrize("dims,width", [(8, 8), (4, 10), (32, 32)])
def test_rotary_kernel(scaling, dims, width):
    ops, rng = _ops(), np.random.default_rng(3)
    from math_utils_b200.parts.position import rotary_frequencies
    rot = {"base": 10000.0, "dims": dims}
    if scaling:
        rot["scaling"] = scaling
    heads, lead = 3, 5                                    # every head's slice sits behind `lead` other entries
    positions = np.array([0, 1, 2, 63, 64, 1000, 40000, 7])
    x = rng.normal(0, 1, (len(positions), heads, lead + width))
    want = plain.rotate(x[..., lead:], positions, rot)
    freqs, mag = rotary_frequencies(dims, rot["base"], scaling)
    pf, pm = plain.rotary_frequencies(rot)
    assert np.allclose(freqs, pf, rtol=1e-12) and abs(mag - pm) < 1e-12
    xd = dev(x.reshape(len(positions), -1))
    out = torch.zeros((len(positions), heads * width), device="cuda")
    ops.rotary(xd[:, lead:], out, dev(positions, torch.int32), dev(np.array(freqs)), mag, heads, dims, width,
               lead + width, width)
    got = out.cpu().numpy().reshape(len(positions), heads, width)
    # float32 angles: an absolute error of position * 2^-24 in the angle
    assert np.abs(got - want).max() < 1e-5 + 40000 * 2.0 ** -23 * 3


def _latent_case(rng, lens, heads, kv_rank, rot_dim, page=64, shuffle=True):
    """Rows of several sequences in pages handed out in a scrambled order."""
    width = kv_rank + rot_dim
    n_pages = sum(-(-n // page) for n in lens) + 3
    order = rng.permutation(n_pages) if shuffle else np.arange(n_pages)
    pages = np.zeros((n_pages, page, width))
    table = np.zeros((len(lens), 8), dtype=np.int32)
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


def _plain_latent(q, rows, kv_rank, scale):
    s = (rows @ q) * scale
    p = np.exp(s - s.max())
    return (p / p.sum()) @ rows[:, :kv_rank]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_rank,rot_dim", [(3, 32, 8), (1, 12, 6), (4, 128, 48), (2, 200, 24)])
@pytest.mark.parametrize("n_splits", [1, 3, 7])
def test_latent_attention_kernel(dtype, heads, kv_rank, rot_dim, n_splits):
    ops, rng = _ops(), np.random.default_rng(4)
    lens = [1, 2, 63, 64, 65, 300]
    seqs, pages, table = _latent_case(rng, lens, heads, kv_rank, rot_dim)
    width, scale = kv_rank + rot_dim, 0.37
    if dtype == torch.bfloat16:                                       # the cache holds what bfloat16 can hold
        pages = dev(pages, dtype).float().cpu().numpy().astype(np.float64)
        seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
    # queries: the last position of every sequence, and some in the middle of the longest
    picks = [(s, n - 1) for s, n in enumerate(lens)] + [(5, 0), (5, 63), (5, 64), (5, 127), (5, 128), (5, 191), (5, 192)]
    q = rng.normal(0, 1, (len(picks), heads, width)) / math.sqrt(width) * 3
    # one far key stands out for the first head of the last query: its score is far above the others
    far = 2
    q[5, 0] = seqs[5][far] * 16.0 / scale / width
    want = np.stack([[_plain_latent(q[i, h], seqs[s][:p + 1], kv_rank, scale) for h in range(heads)]
                     for i, (s, p) in enumerate(picks)])
    assert abs(want[5, 0] - seqs[5][far, :kv_rank]).max() < 0.5 * abs(seqs[5][far, :kv_rank]).max()
    out = torch.zeros((len(picks), heads * kv_rank), device="cuda", dtype=dtype)
    items = len(picks) * heads
    part_o = torch.zeros(items * n_splits * kv_rank, device="cuda")
    part_ml = torch.zeros(items * n_splits * 2, device="cuda")
    args = (dev(q.reshape(len(picks), -1)), dev(pages, dtype), dev(table, torch.int32), 64,
            dev(np.array([p for _, p in picks]), torch.int32), dev(np.array([s for s, _ in picks]), torch.int32),
            heads, kv_rank, scale, out, n_splits, part_o, part_ml)
    ops.latent_attention(*args, tensor_cores=False)
    got = out.float().cpu().numpy().reshape(len(picks), heads, kv_rank)
    assert np.abs(got - want).max() < (2e-5 if dtype == torch.float32 else 2e-2)
    if dtype == torch.bfloat16 and kv_rank % 64 == 0:
        # the same on tensor cores: every query as its sequence's single token (queries and weights rounded to bfloat16)
        out.zero_()
        ops.latent_attention(*args, single_tokens=True, tensor_cores=True)
        got = out.float().cpu().numpy().reshape(len(picks), heads, kv_rank)
        assert np.abs(got - want).max() < 4e-2
        assert np.abs(got[5, 0] - seqs[5][far, :kv_rank]).max() < 0.5 * abs(seqs[5][far, :kv_rank]).max()


@pytest.mark.parametrize("heads,kv_rank,rot_dim", [(3, 64, 16), (6, 128, 16), (16, 256, 32), (40, 64, 0), (2, 512, 64)])
def test_latent_attention_on_tensor_cores_prompt_tiles(heads, kv_rank, rot_dim):
    """Whole prompts of several sequences in one step: tiles of up to 64 tokens, every token its own causal edge."""
    ops, rng = _ops(), np.random.default_rng(8)
    lens = [130, 1, 64, 65, 7]
    seqs, pages, table = _latent_case(rng, lens, heads, kv_rank, rot_dim)
    width, scale = kv_rank + rot_dim, 0.21
    pages = dev(pages, torch.bfloat16).float().cpu().numpy().astype(np.float64)
    seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
    T = sum(lens)
    q = dev(rng.normal(0, 1, (T, heads, width)) / math.sqrt(width) * 4, torch.bfloat16).float().cpu().numpy().astype(np.float64)
    tok_seq = np.repeat(np.arange(len(lens)), lens)
    tok_pos = np.concatenate([np.arange(n) for n in lens])
    tiles, at = [], 0
    for n in lens:
        tiles += [(at + o, min(64, n - o)) for o in range(0, n, 64)]
        at += n
    tiles.sort(key=lambda t: -tok_pos[t[0] + t[1] - 1])
    want = np.stack([[_plain_latent(q[t, h], seqs[tok_seq[t]][:tok_pos[t] + 1], kv_rank, scale) for h in range(heads)]
                     for t in range(T)])
    out = torch.zeros((T, heads * kv_rank), device="cuda", dtype=torch.bfloat16)
    ops.latent_attention(dev(q.reshape(T, -1)), dev(pages, torch.bfloat16), dev(table, torch.int32), 64,
                         dev(tok_pos, torch.int32), dev(tok_seq, torch.int32), heads, kv_rank, scale, out,
                         tiles=dev(np.array(tiles), torch.int32), tensor_cores=True)
    got = out.float().cpu().numpy().reshape(T, heads, kv_rank)
    err = np.abs(got - want).max(axis=(1, 2))
    assert err.max() < 4e-2, f"first wrong token {int(np.argmax(err > 4e-2))} (sequence {tok_seq[np.argmax(err > 4e-2)]}, position {tok_pos[np.argmax(err > 4e-2)]})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_append_kernel(dtype):
    ops, rng = _ops(), np.random.default_rng(5)
    from math_utils_b200.parts.position import rotary_frequencies
    kv_rank, rot_dim, dims, eps = 20, 10, 6, 1e-2
    rot = {"base": 300.0, "dims": dims, "scaling": YARN}
    positions = np.array([0, 63, 64, 130, 5])
    seq_of = np.array([0, 0, 1, 1, 2])
    table = np.array([[4, 1, 0], [2, 6, 5], [3, 0, 0]], dtype=np.int32)
    dkv = dev(rng.normal(0, 2, (5, kv_rank + rot_dim)), dtype)
    x = dkv.float().cpu().numpy().astype(np.float64)
    w = rng.normal(1, 0.2, kv_rank)
    want = np.concatenate([plain.rms_norm(x[:, :kv_rank], w, eps), plain.rotate(x[:, kv_rank:], positions, rot)], axis=1)
    pages = torch.zeros((7, 64, kv_rank + rot_dim), device="cuda", dtype=dtype)
    freqs, mag = rotary_frequencies(dims, rot["base"], rot["scaling"])
    ops.latent_append(dkv, dev(w), eps, dev(np.array(freqs)), mag, dims, kv_rank, rot_dim, dev(positions, torch.int32),
                      dev(seq_of, torch.int32), dev(table, torch.int32), 64, pages)
    got = pages.float().cpu().numpy()
    for t, (p, s) in enumerate(zip(positions, seq_of)):
        row = got[table[s, p // 64], p % 64]
        assert np.abs(row - want[t]).max() < (1e-5 if dtype == torch.float32 else 3e-2)
    assert np.count_nonzero(got.reshape(-1, kv_rank + rot_dim).any(axis=1)) == 5      # no other row was touched
    # the same launch rotates the queries' rotated parts; and alone, for a layer that borrows its cache
    heads, lead = 3, 7
    q = dev(rng.normal(0, 1, (5, heads * (lead + rot_dim))), dtype)
    want_q = plain.rotate(q.float().cpu().numpy().astype(np.float64).reshape(5, heads, lead + rot_dim)[..., lead:], positions, rot)
    for with_rows in (True, False):
        qa = torch.zeros((5, heads * (2 + rot_dim)), device="cuda")
        ops.latent_append(dkv if with_rows else None, dev(w), eps, dev(np.array(freqs)), mag, dims, kv_rank, rot_dim,
                          dev(positions, torch.int32), dev(seq_of, torch.int32), dev(table, torch.int32), 64, pages,
                          queries=(q[:, lead:], lead + rot_dim, qa[:, 2:], 2 + rot_dim, heads))
        got_q = qa.cpu().numpy().reshape(5, heads, 2 + rot_dim)
        assert np.abs(got_q[..., 2:] - want_q).max() < 1e-5 and not got_q[..., :2].any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,tokens", [(6, 2, 70), (3, 3, 5), (5, 1, 33), (40, 4, 200), (8, 2, 1)])
@pytest.mark.parametrize("D,F,tc", [(40, 24, 0), (40, 24, 32), (200, 136, 32), (200, 136, 64)])
def test_routed_experts_kernels(dtype, experts, top, tokens, D, F, tc):
    ops, rng = _ops(), np.random.default_rng(6)
    scale = 1.7
    if tc and dtype != torch.bfloat16:
        pytest.skip("the tensor-core products are bfloat16")
    rnd = lambda *shape, s=1.0: dev(rng.normal(0, s, shape), dtype).float().cpu().numpy().astype(np.float64)
    h = rnd(tokens, D)
    w = {"router": rnd(experts, D, s=0.5), "correction": rng.normal(0, 0.3, experts).astype(np.float32).astype(np.float64)}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = rnd(F, D, s=0.3), rnd(F, D, s=0.3), rnd(D, F, s=0.3)
    mlp = {"router": {"experts": experts, "top": top, "scale": scale}}
    want = plain.routed_ff(h, mlp, w, "")
    P = tokens * top
    max_tiles = P // (tc or ops.moe_tile_rows()) + experts
    expert_of, slot_of, pair_of = (torch.zeros(P, dtype=torch.int32, device="cuda") for _ in range(3))
    tile_info = torch.zeros(3 * max_tiles, dtype=torch.int32, device="cuda")
    n_tiles = torch.zeros(1, dtype=torch.int32, device="cuda")
    weight_of = torch.zeros(P, device="cuda")
    hd = dev(h, dtype)
    ops.moe_route(hd, dev(w["router"]), dev(w["correction"]), top, scale, expert_of, weight_of)
    s = plain.sigmoid(h @ w["router"].T)
    choice = np.argsort(-(s + w["correction"]), axis=1, kind="stable")[:, :top]
    assert (expert_of.cpu().numpy().reshape(tokens, top) == choice).all()
    assert np.abs(weight_of.cpu().numpy().reshape(tokens, top) - np.take_along_axis(s, choice, 1) * scale).max() < 1e-5
    ops.moe_group(expert_of, experts, slot_of, pair_of, tile_info, n_tiles, tc)
    slots = slot_of.cpu().numpy()
    assert sorted(slots.tolist()) == list(range(P)) and (pair_of.cpu().numpy()[slots] == np.arange(P)).all()
    assert (np.diff(expert_of.cpu().numpy()[pair_of.cpu().numpy()]) >= 0).all()     # an expert's slots lie together
    stack = lambda k: dev(np.stack([w[f"e{e}.{k}"] for e in range(experts)]), dtype)
    hidden = torch.zeros((P, F), device="cuda", dtype=dtype)
    ops.moe_gemm(hd, pair_of, top, stack("gate"), stack("up"), tile_info, n_tiles, max_tiles, hidden, tensor_cores=bool(tc), tile_rows=tc)
    y = torch.zeros((P, D), device="cuda")
    ops.moe_gemm(hidden, None, top, stack("down"), None, tile_info, n_tiles, max_tiles, y, tensor_cores=bool(tc), tile_rows=tc)
    out = torch.zeros((tokens, D), device="cuda")
    ops.moe_combine(y, slot_of, weight_of, top, out)
    assert np.abs(out.cpu().numpy() - want).max() < (3e-5 if dtype == torch.float32 else 3e-2) * max(1.0, np.abs(want).max())
    # the sum, Dynamic Tanh and the addition to the stream in one launch
    nw, nb, stream = rng.normal(1, 0.2, D), rng.normal(0, 0.2, D), rng.normal(0, 1, (tokens, D))
    acc = dev(stream)
    ops.moe_combine_tanh(y, slot_of, weight_of, top, dev(nw), dev(nb), dev(np.array([0.7])), acc)
    want2 = acc.cpu().numpy() * 0 + dev(stream).cpu().numpy() + plain.dynamic_tanh(out.cpu().numpy().astype(np.float64), nw, nb, 0.7)
    assert np.abs(acc.cpu().numpy() - want2).max() < 1e-5


def test_sigmoid_gate_kernel():
    ops, rng = _ops(), np.random.default_rng(7)
    o, g = rng.normal(0, 1, (11, 30)), rng.normal(0, 3, (11, 30))
    od = dev(o)
    ops.sigmoid_gate(od, dev(g))
    assert np.abs(od.cpu().numpy() - o * plain.sigmoid(g)).max() < 1e-6


@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16),
                                            (torch.float32, torch.float32)])
@pytest.mark.parametrize("rows,heads,n,k,lead", [(1, 3, 64, 16, 8), (70, 6, 128, 32, 32), (33, 2, 24, 200, 0), (5, 4, 10, 12, 3)])
def test_products_per_head(dtype, out_dtype, rows, heads, n, k, lead):
    """out[t, h] = W[h] x[t, h]: the heads' slices sit `lead` entries apart from one another's ends."""
    ops, rng = _ops(), np.random.default_rng(9)
    xs, os_ = k + lead, n + 5 + (n + 5) % 2
    x = dev(rng.normal(0, 1, (rows, heads * xs)), dtype)
    w = dev(rng.normal(0, 1, (heads, n, k)) / math.sqrt(k), dtype)
    out = torch.zeros((rows, heads * os_), device="cuda", dtype=out_dtype)
    ops.heads_gemm(x, w, out, xs, os_)
    xf, wf = x.float().cpu().numpy().astype(np.float64), w.float().cpu().numpy().astype(np.float64)
    got = out.float().cpu().numpy().reshape(rows, heads, os_)
    for h in range(heads):
        want = xf[:, h * xs: h * xs + k] @ wf[h].T
        assert np.abs(got[:, h, :n] - want).max() < (2e-5 if out_dtype == torch.float32 else 3e-2)
        assert not got[:, h, n:].any()                                      # nothing written between the slices
    if out_dtype == dtype:                                                  # with a gate laid out as the output
        gate = dev(rng.normal(0, 2, (rows, heads * os_)), dtype)
        ops.heads_gemm(x, w, out, xs, os_, gate=gate)
        got = out.float().cpu().numpy().reshape(rows, heads, os_)
        gf = gate.float().cpu().numpy().astype(np.float64).reshape(rows, heads, os_)
        for h in range(heads):
            want = xf[:, h * xs: h * xs + k] @ wf[h].T * plain.sigmoid(gf[:, h, :n])
            assert np.abs(got[:, h, :n] - want).max() < (2e-5 if out_dtype == torch.float32 else 3e-2)
