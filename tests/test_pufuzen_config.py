"""The Pufuzen configuration, its declared tensors, its cache plan and the plain restatement's
own consistency, on the CPU."""
import json

import pytest
import torch

import plain_pufuzen as plain
from tiny_pufuzen import TINY, gru, rotary, windowed
from tokenizer_b200.cache.manager import CachePlan, plan_groups
from tokenizer_b200.config import ConfigError, PufuzenConfig, config_from_dict
from tokenizer_b200.parts import CacheNeed, KVNeed, StateNeed
from tokenizer_b200.parts.model import declared_tensors


def raw(layers):
    return {"architecture": "Pufuzen", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
            "layers": layers}


def test_the_architecture_is_chosen_by_its_name_and_every_size_comes_from_the_file():
    cfg = config_from_dict(raw([gru(40), windowed(3, 8, 6, 10, 12, 5, 0.3, ff=30), rotary(2, 8, 4, 6, 10, 12, 99.0, 0.2)]))
    assert isinstance(cfg, PufuzenConfig)
    spec = cfg.model_spec()
    assert [layer.block for layer in spec.layers] == ["gated_pre_norm_mixer_only", "gated_pre_norm_residual",
                                                      "gated_pre_norm_mixer_only"]
    shapes = {t.name: tuple(t.shape) for t in declared_tensors(spec)}
    assert shapes["embed"] == (50, 24) and shapes["head"] == (50, 24) and shapes["final.norm"] == (24,)
    assert shapes["l0.mix.z"] == (40, 24) and shapes["l0.mix.o"] == (24, 40) and shapes["l0.rg1.b"] == (24,)
    assert "l0.norm2" not in shapes and "l0.rg2" not in shapes
    assert shapes["l1.mix.uq"] == (3 * 8, 10) and shapes["l1.mix.dkv"] == (12, 24) and "l1.mix.sink" not in shapes
    assert shapes["l1.mlp.up"] == (30, 24) and shapes["l1.mlp.act"] == (4,) and shapes["l1.rg2"] == (24, 24)
    assert shapes["l2.mix.uq"] == (2 * (8 + 4), 10) and shapes["l2.mix.dkv"] == (12 + 4, 24)
    assert shapes["l2.mix.uk"] == (2 * 8, 12) and shapes["l2.mix.uv"] == (2 * 6, 12) and shapes["l2.mix.sink"] == (2,)
    assert spec.final_norm.params["gain_scale"] == 2.0
    # a window of n keys is the query and n - 1 keys before it
    assert spec.layers[1].mixer.params["window"] == 4 and spec.layers[2].mixer.params["window"] is None
    assert json.loads(json.dumps(cfg.to_dict()))["architecture"] == "Pufuzen"
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("spoil,word", [
    (lambda r: r["layers"][0].update(type="lstm"), "unknown type"),
    (lambda r: r["layers"][1]["mlp"].update(kind="experts"), "dense"),
    (lambda r: r["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda r: r.update(logit_scale="two"), "logit_scale"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["layers"][1]["mixer"]["mask"].update(size=0), "size"),
    (lambda r: r["layers"][1]["mixer"].update(mask=7), "mask"),
])
def test_a_configuration_that_cannot_be_a_model_is_refused(spoil, word):
    r = raw([gru(40), windowed(3, 8, 6, 10, 12, 5, 0.3, ff=30), rotary(2, 8, 4, 6, 10, 12, 99.0, 0.2)])
    spoil(r)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(r)


def test_the_cache_plan_keeps_one_row_a_token_for_a_latent_and_a_slot_for_a_recurrence():
    needs = [CacheNeed(state=StateNeed((40,))), CacheNeed(kv=KVNeed(1, 48, 6, planes=1)),
             CacheNeed(kv=KVNeed(1, 48, None, planes=1)), CacheNeed(kv=KVNeed(1, 48, 6, planes=1)),
             CacheNeed(kv=KVNeed(1, 48, 6, planes=2))]
    groups, of_call = plan_groups(needs)
    assert of_call == [None, 0, 1, 0, 2] and [g.planes for g in groups] == [1, 1, 2]
    plan = CachePlan(needs, num_pages=6, page_size=8, max_requests=2)
    assert plan.state_calls == [0] and not plan.share_prefixes
    a = plan.open("a")
    plan.reserve(a, 30)
    plan.commit(a, 30)
    # the next query (position 30) reaches back to key 24: the windowed groups keep the page that
    # holds it and gave the three before it back; the causal group kept all four
    assert len(a.pages_held(0)) == 1 and len(a.pages_held(1)) == 4 and len(a.pages_held(2)) == 1
    slot = a.state_slot
    plan.close(a)
    assert plan.open("b").state_slot == slot
    plan.check()


@pytest.mark.parametrize("name", sorted(TINY))
def test_the_tiny_configurations_declare_what_random_weights_write(name, tmp_path):
    from tokenizer_b200 import write_random_model
    cfg, seed, _ = TINY[name]()
    folder = write_random_model(str(tmp_path / name), cfg, seed)
    raw_cfg, weights = plain.load_folder(folder)
    assert set(weights) == {t.name for t in declared_tensors(cfg.model_spec())}
    logits = plain.forward(raw_cfg, weights, [1, 2, 3, 4, 5])
    assert logits.shape == (5, cfg.vocab) and torch.isfinite(logits).all()


def test_the_plain_recurrence_carries_its_state_and_the_plain_attention_its_window_and_sink():
    torch.manual_seed(0)
    f64 = torch.float64
    w = {"m.z": torch.randn(6, 4, dtype=f64), "m.z.b": torch.randn(6, dtype=f64), "m.x": torch.randn(6, 4, dtype=f64),
         "m.x.b": torch.randn(6, dtype=f64), "m.g": torch.randn(6, 4, dtype=f64), "m.o": torch.randn(4, 6, dtype=f64)}
    h = torch.randn(9, 4, dtype=f64)
    whole, end = plain.min_gru(h, w, "m.")
    first, state = plain.min_gru(h[:5], w, "m.")
    second, end2 = plain.min_gru(h[5:], w, "m.", state)
    assert torch.allclose(torch.cat([first, second]), whole) and torch.allclose(end, end2)
    m = {"heads": 2, "dim": 4, "rot_dim": 2, "vdim": 3, "kv_rank": 5}
    a = {"a.dq": torch.randn(6, 4, dtype=f64), "a.dq.norm": torch.ones(6, dtype=f64), "a.uq": torch.randn(12, 6, dtype=f64),
         "a.dkv": torch.randn(7, 4, dtype=f64), "a.dkv.norm": torch.ones(5, dtype=f64), "a.uk": torch.randn(8, 5, dtype=f64),
         "a.uv": torch.randn(6, 5, dtype=f64), "a.o": torch.randn(4, 6, dtype=f64),
         "a.sink": torch.tensor([-1e9, -1e9], dtype=f64)}
    m["scale"] = 0.5
    causal = plain.latent_attention(h, a, "a.", m, 1e-5, rot=(100.0, 2))
    assert torch.allclose(plain.latent_attention(h, a, "a.", m, 1e-5, rot=(100.0, 2), window=9), causal)
    assert torch.allclose(plain.latent_attention(h, a, "a.", m, 1e-5, rot=(100.0, 2), sink=True), causal)
    assert not torch.allclose(plain.latent_attention(h, a, "a.", m, 1e-5, rot=(100.0, 2), window=2), causal)
    a["a.sink"] = torch.tensor([3.0, 0.0], dtype=f64)
    assert not torch.allclose(plain.latent_attention(h, a, "a.", m, 1e-5, rot=(100.0, 2), sink=True), causal)
    # a window of one key: every position sees itself alone, so the output is its own value's projection
    a["a.uq"], a["a.dkv"] = a["a.uq"][:8], a["a.dkv"][:5]        # the same mixer without positional lanes
    alone = plain.latent_attention(h, a, "a.", dict(m, rot_dim=0), 1e-5, window=1)
    c = plain.rms_norm(plain.linear(h, a["a.dkv"])[:, :5], a["a.dkv.norm"], 1e-5)
    assert torch.allclose(alone, plain.linear(plain.linear(c, a["a.uv"]), a["a.o"]))
