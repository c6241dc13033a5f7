"""The Kiruvik design on the CPU: configuration, run order, tensor list, cache needs, and pages that chunks release."""

import copy

import pytest
import torch

from kiruvik_tools import CONFIGS, draw_weights
from quantinfer_b200.cache import CacheManager
from quantinfer_b200.cache.needs import PagedKVNeed, StateNeed
from quantinfer_b200.config import KiruvikConfig, config_from_dict
from quantinfer_b200.engine.model import tensor_needs_of_spec
from quantinfer_b200.errors import ConfigError


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_round_trip_and_tensor_list(name):
    cfg = config_from_dict(CONFIGS[name])
    assert isinstance(cfg, KiruvikConfig)
    assert cfg.to_dict() == CONFIGS[name]
    rebuilt = KiruvikConfig.from_dict(KiruvikConfig(cfg.vocab, cfg.width, cfg.norm_eps, cfg.residual_mult, cfg.layers, cfg.loop).to_dict())
    assert rebuilt == cfg
    needs = tensor_needs_of_spec(cfg.to_model_spec())
    w = draw_weights(CONFIGS[name], 1)
    assert set(needs) == set(w)
    assert all(tuple(needs[k].shape) == tuple(w[k].shape) for k in w)


def test_run_order_of_a_loop_and_its_cache_entries():
    spec = config_from_dict(CONFIGS["P"]).to_model_spec()
    assert [(c.layer, c.reenter) for c in spec.order] == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert [c.cache for c in spec.order] == list(range(8)) and all(c.writes_cache for c in spec.order)
    assert spec.reentry is not None and spec.reentry.weight_name == "loop.in"
    spec = config_from_dict(CONFIGS["Q"]).to_model_spec()
    assert spec.reentry is None and not any(c.reenter for c in spec.order)
    spec = config_from_dict(CONFIGS["R"]).to_model_spec()
    assert [(c.layer, c.reenter) for c in spec.order] == [(0, True), (1, False)] * 2


def test_specs_carry_every_constant_of_the_file():
    spec = config_from_dict(CONFIGS["P"]).to_model_spec()
    a = spec.layers[0].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.chunk, a.position.rotary_dim, a.position.theta) == (3, 3, 10, 6, 9, 4, 300.0)
    assert a.position.pairing == "half_split" and spec.layers[3].mixer.position is None and spec.layers[3].mixer.chunk is None
    s = spec.layers[1].mixer
    assert (s.heads, s.head_dim, s.state, s.groups, s.conv_taps, s.norm_groups, s.norm_eps) == (4, 6, 5, 2, 4, 3, 3e-6)
    f = spec.layers[1].ffn
    assert (f.experts, f.top, f.router_scale, f.expert.intermediate_size, f.expert.limit, f.shared.intermediate_size, f.shared.limit) == (5, 3, 1.7, 12, 0.8, 20, 1.3)
    assert spec.layers[2].ffn.shared is None and spec.layers[3].ffn is None and spec.layers[0].residual_mult == 0.7
    assert spec.layers[0].ffn.activation == "gelu_tanh" and spec.final_norm.kind == "dyt"


@pytest.mark.parametrize("edit, text", [
    (lambda d: d["layers"][0].update(type="conv"), "mixers are"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=2), "multiple of kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=5), "even"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "top <= experts"),
    (lambda d: d["loop"].update(stop=9), "stretch"),
    (lambda d: d["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda d: d.pop("width"), "width"),
])
def test_bad_configurations_are_refused(edit, text):
    d = copy.deepcopy(CONFIGS["P"])
    edit(d)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(d)


def test_pages_of_chunks_a_request_has_left_go_back():
    """Chunks of 12 positions over pages of 4: after 30 positions the next query sits in the chunk that starts at 24,
    so the six pages before it are free again; a group without chunks keeps all its pages."""
    needs = [PagedKVNeed(2, 8, None, 6, 12), PagedKVNeed(2, 8), StateNeed((5,), torch.float32)]
    cm = CacheManager(needs, page_size=4, num_pages=16, max_requests=2, max_seq_len=64)
    assert len(cm.groups) == 2
    chunked = 0 if cm.groups[0].need.chunk else 1
    cm.open("a")
    cm.prepare("a", 30)
    assert cm.free_pages(chunked) == 16 - 8
    cm.commit("a")
    assert cm.free_pages(chunked) == 16 - 2 and cm.free_pages(1 - chunked) == 16 - 8
    assert cm.table_row("a", chunked)[:8] == [-1] * 6 + cm.table_row("a", chunked)[6:8]
    cm.prepare("a", 7)          # through position 36: the chunk that starts at 36 begins on a page's border
    cm.commit("a")
    assert cm.free_pages(chunked) == 16 - 1
    cm.check_invariants()
    cm.close("a")
    assert cm.free_pages(chunked) == 16 and cm.free_pages(1 - chunked) == 16
    k, v = needs[0].pools(4)
    assert k == (2, 4, 8) and v == (2, 4, 6)
