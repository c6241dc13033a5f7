"""The Bebuvik configuration, its description as parts, its tensor list, its cache needs and the cache manager's
handling of them: everything that needs no device."""

import copy

import pytest
import torch

from bebuvik_tools import CONFIGS, draw_weights, write_folder


def test_the_registry_finds_the_design_by_its_one_string():
    from quantinfer_b200.config import BebuvikConfig, architectures, config_from_dict

    assert "Bebuvik" in architectures()
    cfg = config_from_dict(CONFIGS["P"])
    assert isinstance(cfg, BebuvikConfig)
    assert cfg.to_dict() == CONFIGS["P"]
    assert config_from_dict(cfg.to_dict()) == cfg
    again = BebuvikConfig(cfg.vocab, cfg.width, cfg.norm_eps, cfg.layers, cfg.taps, cfg.bigram, cfg.logit_softcap)
    assert config_from_dict(again.to_dict()) == cfg            # the dictionary is rebuilt from the fields alone


def test_every_size_and_constant_reaches_the_spec():
    from quantinfer_b200.config import config_from_dict

    spec = config_from_dict(CONFIGS["P"]).to_model_spec()
    assert (spec.vocab_size, spec.hidden_size, len(spec.layers)) == (211, 44, 4)
    e = spec.embedding
    assert (e.kind, e.buckets, e.mul_prev, e.mul_cur) == ("bigram_embedding", 97, 31, 5)
    assert spec.head.softcap == 7.5 and not spec.head.tied
    m0, m1, m2, m3 = (layer.mixer for layer in spec.layers)
    assert (m0.num_heads, m0.head_dim, m0.rot_dim, m0.value_dim, m0.kv_rank, m0.window) == (3, 10, 4, 12, 18, 9)
    assert m1.shares_latent and m1.window == 21 and not m0.shares_latent
    assert (m2.position.rotary_dim, m2.position.theta, m2.position.pairing) == (4, 500.0, "interleaved")
    assert m2.window is None and m3.window == 5 and m3.num_heads == 5
    assert spec.layers[1].ffn is None and spec.layers[1].conv.names == ("l1.canon1",)
    assert spec.layers[0].conv.taps == 3 and spec.layers[0].conv.names == ("l0.canon1", "l0.canon2")
    assert spec.layers[0].norm.kind == "rmsnorm_scalar" and spec.layers[0].norm.eps == 3e-6
    # layers 1 and 3 read the entries that 0 and 2 write
    assert [(c.layer, c.cache, c.writes_cache) for c in spec.order] == [(0, 0, True), (1, 0, False), (2, 1, True), (3, 1, False)]
    bare = config_from_dict(CONFIGS["R"]).to_model_spec()
    assert bare.embedding.kind == "embedding" and bare.head.softcap is None and bare.layers[0].conv is None


def test_tensor_names_and_shapes():
    from quantinfer_b200.config import config_from_dict
    from quantinfer_b200.engine import tensor_needs_of_spec

    for name, cfg in CONFIGS.items():
        needs = tensor_needs_of_spec(config_from_dict(cfg).to_model_spec())
        w = draw_weights(cfg, 0)
        assert {k: tuple(v.shape) for k, v in needs.items()} == {k: tuple(v.shape) for k, v in w.items()}, name
    needs = tensor_needs_of_spec(config_from_dict(CONFIGS["P"]).to_model_spec())
    assert "l1.mix.dkv" not in needs and "l1.mlp.up" not in needs and "l1.rg2" not in needs and "l1.canon2" not in needs
    assert needs["l0.norm1"].shape == () and needs["bigram"].shape == (98, 44)


@pytest.mark.parametrize("change, message", [
    (lambda d: d["layers"][1]["mixer"].update(kv_from=1), "earlier layer"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "no latent projection"),
    (lambda d: d["layers"][1]["mixer"].update(kv_rank=20), "differ"),
    (lambda d: d["layers"][0].update(type="attention"), "latent_attention"),
    (lambda d: d["layers"][0]["mlp"].update(kind="gated"), "dense"),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=5), "even"),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=8), "within"),
    (lambda d: d["canon"].update(taps=0), "taps"),
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].update(eps=0), "eps"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "mask"),
])
def test_what_the_configuration_refuses(change, message):
    from quantinfer_b200.config import config_from_dict
    from quantinfer_b200.errors import ConfigError

    d = copy.deepcopy(CONFIGS["P"])
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_a_folder_loads_and_a_wrong_one_says_what_is_wrong(tmp_path):
    from quantinfer_b200.config import load_config
    from quantinfer_b200.engine import tensor_needs_of_spec
    from quantinfer_b200.errors import WeightError
    from quantinfer_b200.weights import load_folder, write_model_folder

    cfg = CONFIGS["S"]
    w = draw_weights(cfg, 3)
    folder = write_folder(tmp_path / "ok", cfg, w)
    needs = tensor_needs_of_spec(load_config(folder).to_model_spec())
    got = load_folder(folder, needs)
    assert got["l0.norm1"].shape == () and torch.equal(got["l2.mix.sink"], w["l2.mix.sink"])
    bad = dict(w)
    del bad["l1.mix.uk"]
    bad["l0.mix.sink"] = torch.zeros(3, dtype=torch.bfloat16)
    with pytest.raises(WeightError) as err:
        load_folder(write_folder(tmp_path / "bad", cfg, bad), needs)
    assert "l1.mix.uk" in str(err.value) and "l0.mix.sink" in str(err.value)
    # a folder of random weights for the design loads like any other
    rnd = write_model_folder(tmp_path / "rnd", load_config(folder), seed=5)
    assert set(load_folder(rnd, needs)) == set(needs)


def test_needs_merge_and_the_manager_keeps_pages_for_the_widest_reader():
    from quantinfer_b200.cache import CacheManager, PagedKVNeed, PagedLatentNeed, StateNeed

    a, b = PagedLatentNeed(22, 9), PagedLatentNeed(22, 21)
    assert a.merged(b) == PagedLatentNeed(22, 21) and a.merged(PagedLatentNeed(22, None)).window is None
    assert a.merged(PagedLatentNeed(24, 9)) is None and a.merged(PagedKVNeed(1, 22, 9)) is None
    assert PagedKVNeed(2, 8, 4).merged(PagedKVNeed(2, 8, 6)) == PagedKVNeed(2, 8, 6)
    # one latent entry with a window of 21, one with all positions, one state of fixed size: two groups
    cm = CacheManager([PagedLatentNeed(22, 21), PagedLatentNeed(22, None), StateNeed((2, 44), torch.float32)], page_size=8,
                      num_pages=12, max_requests=3, max_seq_len=96)
    assert len(cm.groups) == 2 and cm.pool_bytes() == 2 * 12 * 8 * 22 * 4
    cm.open("a")
    for n in (5, 30, 1, 1, 20):
        cm.prepare("a", n)
        cm.commit("a")
        cm.check_invariants()
    rc = cm.get("a")
    assert rc.length == 57
    # the next query is at 57 and sees 37..57: blocks 0..3 of the windowed group are free again, none of the other
    assert rc.tables[0][:4] == [-1] * 4 and all(p >= 0 for p in rc.tables[0][4:]) and all(p >= 0 for p in rc.tables[1])
    cm.close("a")
    assert cm.free_pages(0) == 12 and cm.free_pages(1) == 12


def test_the_model_collects_state_entries_for_blocks_and_embedding():
    """What each layer call and the embedding keep of a request is an entry of the cache manager's list."""
    from quantinfer_b200.cache import PagedLatentNeed, StateNeed
    from quantinfer_b200.config import config_from_dict
    from quantinfer_b200.engine.model import Model
    from quantinfer_b200.parts import Runtime

    class NoDevice(Runtime):
        def __post_init__(self):
            self.device = torch.device("cpu")

    spec = config_from_dict(CONFIGS["P"]).to_model_spec()
    model = Model(spec, NoDevice(torch.float32, "cpu"))
    assert model.cache_needs[:2] == [PagedLatentNeed(22, 21), PagedLatentNeed(28, None)]      # widened by their readers
    assert model.call_state_entry == [2, 3, 4, 5] and model.embedding_state_entry == 6
    assert model.cache_needs[2] == StateNeed((2, 44), torch.float32) and model.cache_needs[6] == StateNeed((1,), torch.int32)
    one_tap = Model(config_from_dict(CONFIGS["T"]).to_model_spec(), NoDevice(torch.float32, "cpu"))
    assert one_tap.call_state_entry == [None, None, None]          # a filter of one tap keeps nothing


def test_the_comparison_of_bench_py_describes_two_models_of_equal_layer_sizes():
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    from quantinfer_b200.config import config_from_dict

    for size, z in bench.COMPARE_SIZES.items():
        latent, dense = bench.compare_entries(size)
        lc, dc = config_from_dict(latent["config"]), config_from_dict(dense["config"])
        ls, ds = lc.to_model_spec(), dc.to_model_spec()
        assert (ls.hidden_size, ls.vocab_size, len(ls.layers)) == (ds.hidden_size, ds.vocab_size, len(ds.layers)) == (z["width"], 32768, 4)
        assert ls.layers[0].mixer.num_heads == ds.layers[0].mixer.num_heads == z["heads"]
        assert ds.layers[0].mixer.head_dim == z["dim"] + z["rot"]
        assert [c.writes_cache for c in ls.order] == [True, False, True, False]
        la, da = bench.model_arithmetic(lc, ls), bench.model_arithmetic(dc, ds)
        assert 0.8 < la["weight_bytes"] / da["weight_bytes"] < 1.25            # about the same number of parameters
        assert la["kv_bytes_per_token"] < da["kv_bytes_per_token"] and la["attn_flops"](64) > 0
