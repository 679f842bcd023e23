"""Lusalorn's configuration and plan, the cache entries of a layer with two mixers, and the plain statement's own
properties; no device needed."""
import json

import numpy as np
import pytest
import torch

import plain_lusalorn as plain
from math_utils_b200.cache import SequenceCache
from math_utils_b200.config import ConfigError, LusalornConfig, architecture_for
from math_utils_b200.engine.assemble import collect_tensor_specs
from math_utils_b200.parts import CompositeCacheSpec, RowCacheSpec, StateCacheSpec

ROT = {"base": 1.0e4, "dims": 4}
ATT = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "mask": {"size": 40}, "scale": 0.3, "diff": 0.25, "rot": ROT}
PAR = {"left": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 4, "scale": 0.3, "rot": ROT},
       "right": {"heads": 2, "vdim": 4, "state": 6, "groups": 1, "conv": 3, "norm_groups": 2},
       "left_scale": 0.7, "right_scale": 1.3}
CFG = {"architecture": "Lusalorn", "vocab": 90, "width": 32, "residual_mult": 0.5, "norm": {"eps": 1e-5},
       "embedding": {"bigram": {"buckets": 17, "mul_prev": 5, "mul_cur": 3}},
       "layers": [{"type": "attention", "mixer": ATT, "mlp": {"kind": "dense", "ff": 48}},
                  {"type": "parallel", "mixer": PAR, "mlp": {"kind": "dense", "ff": 48}},
                  {"type": "attention", "mixer": dict(ATT, kv_from=0, mask={"size": 70}), "mlp": None}]}


def test_configuration_and_plan():
    assert architecture_for(CFG).config_class is LusalornConfig
    plan = LusalornConfig.from_json(CFG).plan()
    assert [e.cache_of for e in plan.schedule] == [0, 1, 0]
    # the owner's cache keeps what the borrowing layer's wider window sees
    assert plan.layers[0].mixer.params["cache_window"] == 70 and plan.layers[0].mixer.params["window"] == 40
    assert plan.layers[2].feed_forward.kind == "none"
    assert LusalornConfig.from_json(LusalornConfig.from_json(CFG).to_json()).plan() == plan
    names = {s.name: tuple(s.shape) for s in collect_tensor_specs(plan)}
    assert names == plain.tensor_shapes(CFG)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),            # a parallel layer keeps no such keys
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),            # not an earlier layer
    (lambda c: c["layers"][2]["mixer"].update(dim=16), "kv_from"),               # another key size than its owner's
    (lambda c: c["layers"][1]["mixer"]["right"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda c: c["layers"][0].update(type="latent_attention"), "type"),
    (lambda c: c["embedding"].pop("bigram"), "bigram"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
])
def test_configuration_errors_name_the_key(change, word):
    bad = json.loads(json.dumps(CFG))
    change(bad)
    with pytest.raises(ConfigError, match=word):
        LusalornConfig.from_json(bad)


def test_cache_entries_of_a_layer_with_two_mixers():
    rows, state = RowCacheSpec(24, 0), StateCacheSpec(50)
    specs = [RowCacheSpec(40, 70), CompositeCacheSpec((rows, state)), None, CompositeCacheSpec((rows, None))]
    cache = SequenceCache(specs, 64 * 6, 1024, torch.float32, "cpu", n_slots=3)
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 1
    pair = cache.entry(1)
    assert pair[0].pages.shape == (6, 64, 24) and pair[1].values.shape == (3, 50)
    assert cache.entry(3)[1] is None and cache.entry(3)[0].pages.shape == (6, 64, 24)
    assert cache.entry(3)[0].group == pair[0].group and cache.entry(2) is None
    a = cache.acquire()
    cache.reserve(a, 130)
    cache.commit(a, 130)
    pair[1].values[a] = 3.0
    cache.last_tokens[a] = 7
    kept = cache.snapshot_state([a])
    pair[1].values[a] = 5.0
    cache.last_tokens[a] = 9
    cache.restore_state(kept)
    assert (pair[1].values[a] == 3.0).all() and int(cache.last_tokens[a]) == 7
    cache.release(a)
    assert cache.acquire() == a and (pair[1].values[a] == 0.0).all()          # state starts at zero for the next holder
    assert cache.has_running_state


def test_plain_statement_windows_and_state():
    """The plain statement itself: a token outside every window and state cannot be seen; the first token's row."""
    cfg = json.loads(json.dumps(CFG))
    cfg["layers"] = [cfg["layers"][0], dict(cfg["layers"][2], mixer=dict(ATT, mask={"size": 40}))]     # windows only
    w = plain.random_weights(cfg, 3)
    toks = np.random.default_rng(0).integers(0, 90, 100).tolist()
    base = plain.forward(cfg, w, toks)
    other = list(toks)
    other[10] = (other[10] + 1) % 90
    moved = plain.forward(cfg, w, other)
    # two layers of window 40 carry a token 78 positions far at most; the hashed pair row one more
    assert np.abs(moved[10 + 2 * 39 + 2:] - base[10 + 2 * 39 + 2:]).max() == 0.0
    assert np.abs(moved[10 + 2 * 39 + 1] - base[10 + 2 * 39 + 1]).max() > 0.0
    x = plain.embedding([5, 6], {"embed": np.eye(90), "bigram": np.arange(18 * 90, dtype=float).reshape(18, 90)}, cfg["embedding"]["bigram"])
    assert x[0, 0] == 17 * 90 and x[1, 0] == ((5 * 5 + 6 * 3) % 17) * 90
