"""Rezusun without a GPU: the configuration, the order of layers, the model description and the
tensors it expects, the registry, sizes read from tensor shapes, the cache groups, and the plain
restatement's own identities."""

import json
import os
import tempfile

import numpy as np
import pytest

import plain_rezusun as R
import tiny_rezusun as tiny


def _arch(cfg):
    from kv_cache_optimization_for_llm_b200.registry import resolve_architecture
    return resolve_architecture(cfg)


def test_registry_takes_the_architecture_key_and_lists_the_design():
    from kv_cache_optimization_for_llm_b200.registry import known_architectures
    assert "Rezusun" in known_architectures() and "LlamaForCausalLM" in known_architectures()
    assert _arch(tiny.MIXED).name == "Rezusun"
    assert _arch({"architectures": ["Rezusun"]}).name == "Rezusun"
    with pytest.raises(ValueError):
        _arch({"architecture": "NoSuchDesign"})


def test_layer_order_follows_the_loop():
    from kv_cache_optimization_for_llm_b200.config.model_config import RezusunConfig
    layers = [tiny.general() for _ in range(5)]
    order = lambda loop: RezusunConfig.from_dict(tiny.config(layers, loop=loop)).layer_order()
    assert order(None) == [0, 1, 2, 3, 4]
    assert order({"start": 1, "stop": 3, "times": 3}) == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert order({"start": 0, "stop": 5, "times": 2}) == [0, 1, 2, 3, 4] * 2
    assert order({"start": 4, "stop": 5, "times": 1}) == [0, 1, 2, 3, 4]
    assert order({"start": 2, "stop": 2, "times": 4}) == [0, 1, 2, 3, 4]
    for loop in ({"start": 3, "stop": 2, "times": 2}, {"start": 0, "stop": 6, "times": 2}, {"start": 0, "stop": 1, "times": 0}):
        with pytest.raises(ValueError):
            order(loop)
    # the plain restatement orders them alike
    for loop in (None, {"start": 1, "stop": 3, "times": 3}, {"start": 0, "stop": 5, "times": 2}):
        assert R.layer_order(tiny.config(layers, loop=loop)) == order(loop)


def test_configuration_errors_name_the_key():
    from kv_cache_optimization_for_llm_b200.config.model_config import ConfigError, RezusunConfig
    bad = json.loads(json.dumps(tiny.MIXED))
    del bad["layers"][2]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError, match="kv_rank"):
        RezusunConfig.from_dict(bad)
    bad = json.loads(json.dumps(tiny.MIXED))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError, match="convolution"):
        RezusunConfig.from_dict(bad)
    bad = json.loads(json.dumps(tiny.MIXED))
    bad["layers"][1]["mlp"]["kind"] = "experts"
    with pytest.raises(ConfigError, match="experts"):
        RezusunConfig.from_dict(bad)
    bad = json.loads(json.dumps(tiny.MIXED))
    del bad["norm"]
    with pytest.raises(ConfigError, match="eps"):
        RezusunConfig.from_dict(bad)


def test_description_names_every_tensor_and_each_pass_keeps_its_own_cache():
    from kv_cache_optimization_for_llm_b200.models.spec import expected_weights
    arch = _arch(tiny.MIXED)
    spec = arch.build_spec(arch.parse_config(tiny.MIXED))
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3, 4, 5] and all(e.cache_of is None for e in spec.schedule)
    ew = expected_weights(spec)
    W = tiny.MIXED["width"]
    assert ew["l0.mix.w1"].shape == (6, W) and ew["l0.mix.w2"].shape == (32, 6) and ew["l0.mix.a.b"].shape == (32,)
    assert ew["l1.mix.q.conv"].shape == (24, 4) and ew["l1.mix.v"].shape == (80, W) and ew["l1.mix.b"].shape == (4, W)
    assert ew["l1.mix.norm"].shape == (20,) and ew["l1.mix.g2"].shape == (80, 7) and ew["l1.mix.A_log"].shape == (4,)
    assert ew["l2.mix.dkv"].shape == (16 + 8, W) and ew["l2.mix.uq"].shape == (3 * 24, 20) and ew["l2.mix.sink"].shape == (3,)
    assert ew["l2.mlp.gate.b"].shape == (56,) and ew["l2.ls2"].shape == (W,) and ew["l1.norm2b"].shape == (W,)
    assert "l0.norm2" not in ew and "l0.mlp.gate" not in ew and "l0.ls2" not in ew      # no feed-forward there
    assert ew["embed"].shape == (101, W) and ew["head"].shape == (101, W) and ew["final.norm"].shape == (W,)
    # matrices take the compute type; what enters 32-bit arithmetic stays 32-bit
    assert ew["l2.mix.uk"].kind == "matrix" and ew["l2.mix.sink"].kind == "bias" and ew["l0.mix.norm"].kind == "vector"


def test_ranks_come_from_tensor_shapes_when_the_file_leaves_them_out():
    from kv_cache_optimization_for_llm_b200.weights.loader import stored_shapes
    folder = tempfile.mkdtemp(prefix="kvb200_rzc_")
    tiny.write_model(folder, tiny.MIXED, seed=0)
    bare = json.loads(json.dumps(tiny.MIXED))
    for layer in bare["layers"]:
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
    arch = _arch(bare)
    cfg = arch.parse_config(bare)
    with pytest.raises(ValueError, match="decay_rank"):
        arch.build_spec(cfg)
    full = arch.complete(cfg, stored_shapes(folder))
    assert full.layers[0].mixer["decay_rank"] == 6 and full.layers[1].mixer["gate_rank"] == 7
    assert full.layers[4].mixer["decay_rank"] == 9
    arch.build_spec(full)


def test_cache_groups_state_slots_and_single_plane_pages():
    """The two attention layers keep rows of different width, so each gets a group of one plane; the
    layer in the loop has two passes, each with pages of its own; every delta pass has its own state."""
    import torch
    from kv_cache_optimization_for_llm_b200.cache.paged_cache import PagedCache
    from kv_cache_optimization_for_llm_b200.cache.specs import PagedKVSpec, SlotStateSpec
    specs = [SlotStateSpec((10,)), PagedKVSpec(1, 24, None, planes=1), PagedKVSpec(1, 24, None, planes=1),
             PagedKVSpec(1, 14, None, planes=1), PagedKVSpec(2, 16, None), SlotStateSpec((6,))]
    cache = PagedCache(specs, [None] * 6, page_size=4, num_pages=5, num_slots=2, max_model_len=20,
                       dtype=torch.bfloat16, device="cpu")
    assert cache.group_entries == [2, 1, 1] and sorted(cache.states) == [0, 5]
    assert cache.kv[0].shape == (2, 1, 6, 1, 4, 24) and cache.kv[2].shape == (1, 2, 6, 2, 4, 16)
    b = cache.binding(2)
    assert b.v is None and b.k.shape == (6, 1, 4, 24) and b.group == 0
    assert cache.binding(4).v is not None
    assert cache.bytes_per_page() == 2 * (2 * 24 * 4 + 14 * 4 + 2 * 2 * 16 * 4)
    assert PagedCache.bytes_per_token(specs, [None] * 6, torch.bfloat16) == 2 * (24 + 24 + 14 + 64)
    assert cache.states[0].shape == (3, 10)


def test_plain_rotation_sink_and_convolution():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 2, 8))
    # position 0 turns nothing; dimensions beyond `dims` never turn; a turn keeps each pair's length
    y = R.rotate_interleaved(x, np.arange(5), 100.0, 4)
    assert np.array_equal(y[0], x[0]) and np.array_equal(y[..., 4:], x[..., 4:])
    assert np.allclose(y[..., 0] ** 2 + y[..., 1] ** 2, x[..., 0] ** 2 + x[..., 1] ** 2)
    assert np.allclose(y[3, 1, 2], x[3, 1, 2] * np.cos(3 * 0.1) - x[3, 1, 3] * np.sin(3 * 0.1))
    # a sink far below every score changes nothing; a sink far above takes all the weight
    q, k, v = rng.normal(size=(6, 4)), rng.normal(size=(6, 4)), rng.normal(size=(6, 3))
    plain = R.sink_softmax_attention(q, k, v, 0.5, -1e9)
    assert np.allclose(plain[0], v[0]) and np.abs(R.sink_softmax_attention(q, k, v, 0.5, 50.0)).max() < 1e-15
    one = R.sink_softmax_attention(q[:1], k[:1], v[:1], 0.5, float(q[0] @ k[0]) * 0.5)
    assert np.allclose(one[0], v[0] / 2)            # a sink as large as the only score halves it: it counts once
    # the convolution's last tap weighs the token itself and nothing later leaks in
    taps = rng.normal(size=(3, 4))
    c = R.short_conv(rng.normal(size=(9, 3)), taps)
    x2 = rng.normal(size=(9, 3))
    c2 = R.short_conv(x2, taps)
    assert np.allclose(c2[0], x2[0] * taps[:, 3]) and np.allclose(c2[1], x2[1] * taps[:, 3] + x2[0] * taps[:, 2])
    assert c.shape == (9, 3)


def test_plain_gated_rule_is_the_shared_update():
    rng = np.random.default_rng(0)
    T, Dk, Dv = 12, 6, 5
    g, beta = rng.uniform(0.3, 1.0, (T, Dk)), rng.uniform(0, 1, T)
    k, v, q = rng.normal(size=(T, Dk)), rng.normal(size=(T, Dv)), rng.normal(size=(T, Dk))
    a = R.gated_delta_scan(g, beta, k, v, q)
    b = R.delta_state_scan(g, beta[:, None] * k, k * g, k, beta[:, None] * v, q)
    assert np.abs(a - b).max() < 1e-12


def test_random_model_folder_for_the_design():
    """The framework's own random-weights mode writes a folder that reads back with every tensor."""
    from kv_cache_optimization_for_llm_b200.models.spec import expected_weights
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    from kv_cache_optimization_for_llm_b200.weights.loader import check_and_load
    folder = tempfile.mkdtemp(prefix="kvb200_rzc_")
    write_random_model(folder, tiny.MIXED, seed=3, std=0.1, storage_dtype="bfloat16")
    arch = _arch(tiny.MIXED)
    got = check_and_load(folder, expected_weights(arch.build_spec(arch.parse_config(tiny.MIXED))))
    assert abs(float(got["l2.norm1"].float().mean()) - 1.0) < 0.1 and abs(float(got["l2.mix.sink"].float().mean())) < 0.3
    assert os.path.exists(os.path.join(folder, "config.json"))
