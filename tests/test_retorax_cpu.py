"""Retorax without a GPU: its configuration, its tensor declarations, and the engine's host
side (cache manager, batch packing, step function) driven through the plain kernel references
against the plain implementation of the whole design."""
import random

import pytest
import torch

import retorax_tiny as rx
import schedules
from plain_ops import PlainOps
from rvllm_b200.cache import CacheManager
from rvllm_b200.config import config_from_dict
from rvllm_b200.config.registry import architecture
from rvllm_b200.engine import ModelRunner, load_model, make_cache
from rvllm_b200.errors import ConfigError
from rvllm_b200.parts.base import PagedNeed
from rvllm_b200.parts.model import param_decls


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("rx"))
    return {n: rx.write(root, n) for n in rx.CONFIGS}


def test_config_round_trip_and_errors():
    for name in rx.CONFIGS:
        cfg = config_from_dict(rx.config(name))
        assert config_from_dict(cfg.to_dict()) == cfg
        assert cfg.architecture == "Retorax"
    bad = rx.config("A")
    bad["layers"][2]["mixer"]["kv_from"] = 0                  # a recurrence has no keys
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = rx.config("A")
    bad["layers"][1]["mixer"]["rot"]["dims"] = 34             # more than the head has
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = rx.config("B")
    bad["layers"][0]["mixer"]["heads"] = 6                    # not a multiple of the kv heads
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = rx.config("B")
    del bad["layers"][1]["mixer"]["width"]
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_declared_tensors():
    cfg = config_from_dict(rx.config("A"))
    decls = param_decls(architecture("Retorax").build_spec(cfg))
    assert decls["embed"].shape == (300, 96)
    assert decls["l0.mix.z"].shape == (80, 96) and decls["l0.mix.o"].shape == (96, 80)
    assert decls["l0.mix.z.b"].shape == (80,)
    assert decls["l1.mix.q"].shape == (6 * 32, 96) and decls["l1.mix.v"].shape == (2 * 16, 96)
    assert decls["l1.mix.g"].shape == (6 * 16, 96) and decls["l1.mix.o"].shape == (96, 6 * 16)
    assert decls["l1.mix.talk"].shape == (6, 6) and decls["l1.mix.sink"].shape == (6,)
    assert "l2.mix.k" not in decls and "l2.mix.v" not in decls and "l2.mix.q" in decls
    assert "l2.mlp.up" not in decls and "l2.norm2" not in decls and "l2.norm1b.b" in decls
    assert decls["l4.mlp.act"].shape == (2,)
    assert decls["final.norm.b"].shape == (96,)


def test_cache_groups_and_reach(folders):
    model, _ = load_model(folders["A"], "float32", "cpu", PlainOps())
    needs = model.cache_needs()
    # layer 2 reads layer 1's pages with a larger chunk: the owner's pages are kept
    assert needs[1] == PagedNeed(2, 32, None, None, 16) and needs[2] is None and needs[4] is None
    model, _ = load_model(folders["B"], "float32", "cpu", PlainOps())
    needs = model.cache_needs()
    assert needs[0] == PagedNeed(4, 16, None, 7, 48) and needs[3] == PagedNeed(1, 24, None, 33, 8)
    cache = make_cache(model, 4, 32, 2)
    assert len(cache.groups) == 2 and sorted(cache.states) == [1]
    assert cache.groups[0].k.shape[-1] == 16 and cache.groups[0].v.shape[-1] == 48


def test_pages_of_finished_chunks_come_back():
    cache = CacheManager([PagedNeed(1, 8, None, 10)], [None], 4, 16, 2, allocate=False)
    cache.add("a")
    assert cache.reserve("a", 9)
    cache.advance("a", 9)                   # the next query (9) still sees 0..8
    assert cache.groups[0].pool.in_use == 3
    assert cache.reserve("a", 13)
    cache.advance("a", 10)                  # position 10 opens the second chunk: pages 0, 1 go
    assert list(cache.requests["a"].tables[0])[:2] == [-1, -1]
    cache.advance("a", 13)
    assert cache.groups[0].pool.in_use == 2     # pages 2 (positions 8..11) and 3
    cache.advance("a", 13)
    cache.check()
    cache.free("a")
    assert cache.groups[0].pool.in_use == 0


@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
@pytest.mark.parametrize("schedule", ["whole", "tail_decode", "portions", "mixed"])
def test_engine_host_side_under_every_cut(folders, name, schedule):
    model, _ = load_model(folders[name], "float32", "cpu", PlainOps())
    vocab = rx.config(name)["vocab"]
    rng = random.Random(5)
    reqs = {f"q{i}": [rng.randrange(vocab) for _ in range(n)]
            for i, n in enumerate((61, 2, 35, 1, 90, 17))}
    steps = schedules.tail_decode(reqs, 12) if schedule == "tail_decode" else \
        getattr(schedules, schedule)(reqs)
    page = 4
    cache = make_cache(model, page, schedules.tokens_held(steps, 64) // page, 4)
    runner = ModelRunner(model, cache, PlainOps())
    got = schedules.replay(runner, steps)
    for rid, ids in reqs.items():
        ref = rx.plain_logits(folders[name], name, ids).to(torch.float32)
        for p in range(len(ids)):
            assert torch.allclose(got[(rid, p)], ref[p], atol=3e-5, rtol=0), (rid, p)
    assert not cache.requests and all(g.pool.in_use == 0 for g in cache.groups)
    if name == "B" and schedule != "whole":
        # chunks of 7 positions with pages of 4: finished chunks gave their pages back
        assert cache.groups[0].pool.high_water < sum(-(-len(v) // page) for v in reqs.values())
