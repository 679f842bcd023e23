"""Forisun without a device: config.json -> plan, the tensor list, the registry, frequency tables,
and the bookkeeping of a cache of latent rows."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_forisun as plain
from math_utils_b200.cache import SequenceCache
from math_utils_b200.config import ConfigError, ForisunConfig, architecture_for, load_config
from math_utils_b200.engine.assemble import collect_tensor_specs
from math_utils_b200.parts import RowCacheSpec
from math_utils_b200.parts.position import rotary_frequencies
from math_utils_b200.weights import write_random_model

ROT = {"base": 5000.0, "dims": 6, "scaling": {"factor": 3.0, "original": 100, "fast": 8.0, "slow": 0.5}}
MIX = {"heads": 2, "dim": 5, "rot_dim": 8, "vdim": 7, "kv_rank": 12, "scale": 0.3, "rot": ROT}
CFG = {"architecture": "Forisun", "vocab": 99, "width": 24, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-4},
       "layers": [{"type": "latent_attention", "mixer": MIX, "mlp": {"kind": "dense", "ff": 40}},
                  {"type": "latent_attention", "mixer": dict(MIX, heads=3), "mlp": None},
                  {"type": "latent_attention", "mixer": dict(MIX, kv_from=0, dim=4),
                   "mlp": {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 4, "top": 2, "scale": 2.0}}}]}


def test_registry_finds_the_design_by_its_own_key():
    assert architecture_for(CFG).config_class is ForisunConfig
    with pytest.raises(ConfigError):
        architecture_for({"architecture": "Nobody"})


def test_plan_and_tensor_list_agree_with_the_plain_statement():
    plan = ForisunConfig.from_json(CFG).plan()
    specs = {s.name: tuple(s.shape) for s in collect_tensor_specs(plan)}
    assert specs == {k: tuple(v) for k, v in plain.tensor_shapes(CFG).items()}
    assert [(e.layer, e.cache_of) for e in plan.schedule] == [(0, 0), (1, 1), (2, 0)]
    assert plan.layers[0].mixer.params["own_kv"] and not plan.layers[2].mixer.params["own_kv"]
    assert plan.layers[1].feed_forward.kind == "none" and plan.layers[2].feed_forward.kind == "routed_experts"
    assert plan.embedding.params["scale"] == 1.5 and plan.embedding_norm.kind == "dynamic_tanh"


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1, kv_rank=16), "kv_from"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][0].update(type="other"), "type"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_bad_configurations_name_their_key(change, word):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        ForisunConfig.from_json(cfg).plan()
    assert word in str(e.value)


def test_random_model_folder_round_trips(tmp_path):
    d = write_random_model(str(tmp_path / "m"), CFG, seed=3)
    arch, config, plan = load_config(d)
    assert config.to_json()["layers"] == CFG["layers"]
    from math_utils_b200.weights.safetensors import SafetensorsFile
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    assert {n: tuple(f.tensors[n].shape) for n in f.names()} == {k: tuple(v) for k, v in plain.tensor_shapes(CFG).items()}
    assert tuple(f.read("l0.norm1.alpha").shape) == ()


@pytest.mark.parametrize("rot", [ROT, {"base": 2e5, "dims": 24, "scaling": {"factor": 6.0, "original": 4096, "fast": 24.0, "slow": 2.0}},
                                 {"base": 100.0, "dims": 4}, {"base": 10.0, "dims": 0}])
def test_frequency_tables(rot):
    freqs, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    want, wmag = plain.rotary_frequencies(rot)
    assert len(freqs) == rot["dims"] // 2 and np.allclose(freqs, want, rtol=1e-13) and abs(mag - wmag) < 1e-13
    if "scaling" in rot:
        f = rot["scaling"]["factor"]
        assert abs(freqs[0] - 1.0) < 1e-12 and abs(freqs[-1] * f - rot["base"] ** (-(rot["dims"] - 2) / rot["dims"])) < 1e-12 * f


def test_row_cache_groups_and_pages():
    specs = [RowCacheSpec(20), RowCacheSpec(14), None, RowCacheSpec(20)]
    cache = SequenceCache(specs, max_tokens=64 * 6, max_positions=1024, dtype=torch.float32, device="cpu", n_slots=3)
    assert len(cache.kv_groups) == 2
    assert cache.entry(0).pages.shape == (6, 64, 20) and cache.entry(1).pages.shape == (6, 64, 14)
    assert cache.entry(3).group == cache.entry(0).group and cache.entry(2) is None
    a, b = cache.acquire(), cache.acquire()
    cache.reserve(a, 130); cache.commit(a, 130)
    cache.reserve(b, 1); cache.commit(b, 1)
    assert cache.free_pages(0) == 2 and cache.free_pages(1) == 2
    held = set(cache.block_table_rows(0, [a])[0][:3].tolist())
    cache.release(a)
    c = cache.acquire()
    cache.reserve(c, 192); cache.commit(c, 192)
    assert held == set(cache.block_table_rows(0, [c])[0][:3].tolist())       # the freed pages are the ones used again
    assert cache.free_pages(0) == 2 and cache.length(c) == 192
