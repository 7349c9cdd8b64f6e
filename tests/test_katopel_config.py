"""The Katopel configuration on the CPU: what it reads, what it refuses, the order of a looped
stack, the tensors it declares, the cache groups and the pages a chunked group gives back."""
import copy

import pytest

from tiny_katopel import TINY, attention, config, delta, dense, moe, parallel
from tokenizer_b200.cache.manager import CachePlan
from tokenizer_b200.config import ConfigError, KatopelConfig, config_from_dict
from tokenizer_b200.parts.base import CacheNeed, KVNeed, StateNeed
from tokenizer_b200.parts.model import declared_tensors


def test_the_registry_finds_the_design_by_its_name():
    cfg, _, _ = TINY["a"]()
    again = config_from_dict(cfg.to_dict())
    assert isinstance(again, KatopelConfig) and again.to_dict() == cfg.to_dict()


def test_a_looped_stack_is_called_again_with_caches_of_its_own():
    cfg, _, _ = TINY["a"]()
    order = cfg.model_spec().order
    assert [c.layer for c in order] == [0, 1, 2, 1, 2, 1, 2]
    assert all(c.cache is None for c in order)
    entries = [(at, c.before.params["index"], c.before.params["add_embedding"]) for at, c in enumerate(order)
               if c.before is not None]
    assert entries == [(1, 0, False), (3, 1, True), (5, 2, True)]


def test_no_loop_and_a_loop_of_one_pass():
    cfg, _, _ = TINY["b"]()
    spec = cfg.model_spec()
    assert [c.layer for c in spec.order] == [0, 1] and all(c.before is None for c in spec.order)
    assert "loop.step" not in {t.name for t in declared_tensors(spec)}
    cfg, _, _ = TINY["c"]()
    spec = cfg.model_spec()
    assert [c.layer for c in spec.order] == [0, 1] and spec.order[0].before.params["passes"] == 1
    assert ("loop.step", (1, 50)) in {(t.name, tuple(t.shape)) for t in declared_tensors(spec)}


def test_declared_tensors_follow_the_sizes():
    cfg, _, _ = TINY["a"]()
    shapes = {t.name: tuple(t.shape) for t in declared_tensors(cfg.model_spec())}
    assert shapes["embed"] == (301, 96) and shapes["loop.step"] == (3, 96)
    assert shapes["l0.mix.left.q"] == (4 * 32, 96) and shapes["l0.mix.left.k"] == (32, 96)
    assert shapes["l0.mix.left.v"] == (16, 96) and shapes["l0.mix.left.o"] == (96, 4 * 16)
    assert shapes["l0.mix.left.q.b"] == (128,)
    assert shapes["l0.mix.right.q"] == (16, 96) and shapes["l0.mix.right.v"] == (48, 96)
    assert shapes["l0.mix.right.v.conv"] == (48, 3) and shapes["l0.mix.right.norm"] == (24,)
    assert shapes["l1.mix.q.conv"] == (72, 2) and shapes["l1.mix.A_log"] == (3,) and shapes["l1.mix.b"] == (3, 96)
    assert shapes["l1.mlp.e5.down"] == (96, 40) and shapes["l1.mlp.router"] == (6, 96)
    assert shapes["l1.mlp.shared.gate"] == (56, 96) and shapes["l1.mlp.shared.sg"] == (1, 96)
    assert shapes["l0.mlp.gate"] == (136, 96) and shapes["l0.norm1b.b"] == (96,) and shapes["final.norm.b"] == (96,)
    assert not any(name.startswith("l2.mlp") or name.startswith("l2.norm2") for name in shapes)
    assert "head" not in shapes          # logits come from the embedding table


@pytest.mark.parametrize("change,word", [
    (lambda r: r["layers"][0].update(type="other"), "unknown type"),
    (lambda r: r["layers"][1]["mixer"].update(heads=4), "do not divide"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=34), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "experts"),
    (lambda r: r["layers"][1]["mlp"].update(kind="sparse"), "dense or moe"),
    (lambda r: r["loop"].update(stop=4), "loop"),
    (lambda r: r.pop("norm"), "norm"),
])
def test_what_the_configuration_refuses(change, word):
    raw = copy.deepcopy(TINY["a"]()[0].to_dict())
    change(raw)
    with pytest.raises(ConfigError, match=word):
        KatopelConfig.from_dict(raw)


def test_chunked_keys_form_a_group_of_their_own_and_give_pages_back():
    """Two calls keep keys in chunks of 24, one keeps all keys of the same shape; a request's pages
    wholly before the chunk of its next position go back to the pool."""
    needs = [CacheNeed(kv=KVNeed(2, 32, None, chunk=24), state=StateNeed((8,))), CacheNeed(kv=KVNeed(2, 32)),
             CacheNeed(state=StateNeed((4,))), CacheNeed(kv=KVNeed(2, 32, None, chunk=24))]
    plan = CachePlan(needs, num_pages=16, page_size=8, max_requests=2)
    assert [(g.chunk, g.calls) for g in plan.groups] == [(24, [0, 3]), (None, [1])]
    assert plan.state_calls == [0, 2] and not plan.share_prefixes
    cache = plan.open("r")
    plan.reserve(cache, 30)
    plan.commit(cache, 30)              # next position 30: chunk 24 .. 47, block 3 on
    assert cache.tables[0] == [-1, -1, -1, 0 + cache.tables[0][3]] and all(p >= 0 for p in cache.tables[1])
    assert plan.allocators[0].available == 15 and plan.allocators[1].available == 12
    plan.reserve(cache, 20)             # positions 30 .. 49 cross into the chunk that starts at 48
    plan.commit(cache, 20)              # next position 50: chunk 48 .., block 6 on
    assert [p >= 0 for p in cache.tables[0]] == [False] * 6 + [True]
    plan.check()
    plan.close(cache)
    assert all(a.available == 16 for a in plan.allocators)
