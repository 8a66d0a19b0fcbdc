"""Bizenex without a GPU: its configuration, its tensor declarations, and the engine's host
side (cache manager, batch packing, step function) driven through the plain kernel references
against the plain implementation of the whole design."""
import random

import pytest
import torch

import bizenex_tiny as bz
import schedules
from plain_ops import PlainOps
from rvllm_b200.config import config_from_dict
from rvllm_b200.config.registry import architecture
from rvllm_b200.engine import ModelRunner, load_model, make_cache
from rvllm_b200.errors import ConfigError
from rvllm_b200.parts.base import PagedNeed
from rvllm_b200.parts.model import param_decls


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("bz"))
    return {n: bz.write(root, n) for n in bz.CONFIGS}


def test_config_round_trip_and_errors():
    for name in bz.CONFIGS:
        cfg = config_from_dict(bz.config(name))
        assert config_from_dict(cfg.to_dict()) == cfg
        assert cfg.architecture == "Bizenex"
    bad = bz.config("A")
    bad["layers"][2]["mixer"]["kv_from"] = 1                  # not a latent layer
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = bz.config("A")
    bad["layers"][4]["mixer"]["kv_from"] = 2                  # a reader has no rows of its own
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = bz.config("A")
    bad["layers"][2]["mixer"]["kv_rank"] = 16                 # another rank than its source
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = bz.config("B")
    bad["layers"][0]["mixer"]["kv_heads"] = 3                 # does not divide the heads
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = bz.config("B")
    bad["layers"][0]["mlp"]["router"]["groups"]["count"] = 2  # 9 experts in 2 groups
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = bz.config("A")
    bad["layers"][0]["mlp"]["router"]["top"] = 5              # 2 groups of 2 cannot give 5
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = bz.config("B")
    del bad["layers"][1]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_declared_tensors():
    cfg = config_from_dict(bz.config("A"))
    decls = param_decls(architecture("Bizenex").build_spec(cfg))
    assert decls["embed"].shape == (300, 96) and decls["head"].shape == (300, 96)
    assert decls["l0.mix.q"].shape == (4 * 16, 96) and decls["l0.mix.dkv"].shape == (32, 96)
    assert decls["l0.mix.dkv.norm"].shape == (32,) and decls["l0.mix.uk"].shape == (64, 32)
    assert decls["l0.mix.uv"].shape == (4 * 24, 32) and decls["l0.mix.sink"].shape == (4,)
    assert decls["l0.mix.g"].shape == (96, 96) and decls["l0.mix.o"].shape == (96, 96)
    assert decls["l0.mlp.router"].shape == (6, 96) and decls["l0.mlp.e5.down"].shape == (96, 64)
    assert "l0.mlp.e6.gate" not in decls
    assert decls["l1.mix.k"].shape == (2 * 32, 96) and decls["l1.mix.v"].shape == (2 * 16, 96)
    assert decls["l1.mix.o"].shape == (96, 6 * 16) and "l1.mix.sink" not in decls
    assert "l2.mix.dkv" not in decls and "l2.mix.dkv.norm" not in decls
    assert decls["l2.mix.uk"].shape == (2 * 24, 32) and "l2.norm2" not in decls
    assert decls["final.norm.b"].shape == (96,) and decls["l3.norm2.b"].shape == (96,)


def test_cache_holds_one_latent_row_a_token(folders):
    model, _ = load_model(folders["A"], "float32", "cpu", PlainOps())
    needs = model.cache_needs()
    assert needs[0] == PagedNeed(1, 32, values=False) and needs[2] is None and needs[4] is None
    assert needs[1] == PagedNeed(2, 32, v_head_dim=16) and needs[3] == PagedNeed(3, 16, v_head_dim=32)
    cache = make_cache(model, 4, 32, 2)
    assert len(cache.groups) == 3
    assert cache.groups[0].k.shape[-2:] == (1, 32) and cache.groups[0].v.numel() == 0
    # 32 numbers for the latent layer and its two readers, keys and values for the others
    assert cache.bytes_per_token() == 4 * (32 + 2 * (32 + 16) + 3 * (16 + 32))


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
def test_engine_host_side_under_every_cut(folders, name, schedule):
    model, _ = load_model(folders[name], "float32", "cpu", PlainOps())
    vocab = bz.config(name)["vocab"]
    rng = random.Random(5)
    reqs = {f"q{i}": [rng.randrange(vocab) for _ in range(n)]
            for i, n in enumerate((61, 2, 35, 1, 90, 17))}
    steps = schedules.tail_decode(reqs, 12) if schedule == "tail_decode" else \
        getattr(schedules, schedule)(reqs)
    page = 4
    cache = make_cache(model, page, schedules.tokens_held(steps, 64) // page, 4)
    runner = ModelRunner(model, cache, PlainOps())
    got = schedules.replay(runner, steps)
    tensors = bz.read_tensors(folders[name])
    for rid, ids in reqs.items():
        ref = bz.plain_logits(folders[name], name, ids, tensors=tensors).to(torch.float32)
        for p in range(len(ids)):
            assert torch.allclose(got[(rid, p)], ref[p], atol=3e-5, rtol=0), (rid, p)
    assert not cache.requests and all(g.pool.in_use == 0 for g in cache.groups)
