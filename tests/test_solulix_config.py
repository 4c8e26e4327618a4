"""Solulix without a GPU: the configuration, the model description and its tensor names, the cache
manager's kept first pages, and the plain restatement checked against second formulations."""

import numpy as np
import pytest

import plain_solulix as S
import tiny_solulix as tiny


def _parse(cfg):
    from kv_cache_optimization_for_llm_b200.registry import resolve_architecture
    arch = resolve_architecture(cfg)
    return arch, arch.parse_config(cfg)


def test_description_names_every_tensor_and_schedules_every_pass():
    arch, cfg = _parse(tiny.MIXED)
    spec = arch.build_spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3, 1, 2, 3, 4]
    starts = [(i, e.before.params["index"], e.before.params["add_embedding"]) for i, e in enumerate(spec.schedule) if e.before]
    assert starts == [(1, 0, False), (4, 1, True)]
    assert [layer.block for layer in spec.layers] == ["parallel", "parallel", "parallel_mixer_only", "parallel", "parallel"]
    names = tiny.expected(tiny.MIXED)
    assert names["loop.step"].shape == (2, 48) and names["embed.norm"].shape == (48,)
    assert names["l1.mlp.router"].shape == (6, 48) and names["l1.mlp.correction"].shape == (6,)
    assert names["l1.mlp.e4.down"].shape == (48, 12) and names["l1.mlp.shared.up"].shape == (20, 48)
    assert "l4.mlp.shared.up" not in names and "l4.mlp.e3.up" not in names and "l2.mlp.up" not in names
    assert names["l4.mix.q.conv"].shape == (6 * 24, 4) and names["l4.mix.v"].shape == (8, 48)
    assert names["l0.mix.A_log"].shape == (4,) and names["l0.mix.a"].shape == (4, 48) and names["l0.mix.norm"].shape == (20,)
    assert names["l0.mix.q"].shape == (24, 48) and names["l0.mix.v"].shape == (80, 48)


def test_a_model_without_a_loop_has_no_pass_starts():
    cfg = tiny.config([tiny.attention(), tiny.delta(mlp=tiny.dense())])
    arch, parsed = _parse(cfg)
    spec = arch.build_spec(parsed)
    assert all(e.before is None for e in spec.schedule) and "loop.step" not in tiny.expected(cfg)


@pytest.mark.parametrize("breakage,needle", [
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["mask"].pop("keep_first"), "keep_first"),
    (lambda c: c["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][1]["mlp"]["router"].pop("top"), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "sparse"),
    (lambda c: c["layers"][1].update(type="convolution"), "convolution"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "chooses"),
])
def test_configuration_errors_name_the_key(breakage, needle):
    import copy
    from kv_cache_optimization_for_llm_b200.config import ConfigError
    cfg = copy.deepcopy(tiny.MIXED)
    breakage(cfg)
    with pytest.raises(ConfigError, match=needle):
        _parse(cfg)


def test_cache_manager_keeps_the_pages_of_the_first_tokens():
    from kv_cache_optimization_for_llm_b200.cache.paged_cache import host_runtime
    H = host_runtime()
    m = H.CacheManager([H.GroupSpec(4, 6, 5)], [12], 2)       # pages of 4, window 6, the first 5 tokens stay
    m.admit(1)
    assert m.extend(1, 30)
    m.advance(1, 30)
    table = list(m.block_table(1, 0))
    # tokens 0..4 live on pages 0 and 1; the next query (position 30) reads keys from 25 on: page 6 onwards
    assert [p >= 0 for p in table] == [True, True, False, False, False, False, True, True]
    assert m.free_pages(0) == 12 - 4 and m.check() == ""
    assert m.extend(1, 41)
    m.advance(1, 41)
    assert [p >= 0 for p in m.block_table(1, 0)][:3] == [True, True, False]
    m.release(1)
    assert m.free_pages(0) == 12 and m.check() == ""
    # without kept tokens the same window gives the first pages back
    m2 = H.CacheManager([H.GroupSpec(4, 6)], [12], 2)
    m2.admit(1)
    m2.extend(1, 30)
    m2.advance(1, 30)
    assert [p >= 0 for p in m2.block_table(1, 0)][:2] == [False, False]


def test_a_mixer_may_ask_for_pages_and_a_state_slot():
    import torch
    from kv_cache_optimization_for_llm_b200.cache.paged_cache import PagedCache
    from kv_cache_optimization_for_llm_b200.cache.specs import PagedKVSpec, PagedWithStateSpec, SlotStateSpec
    both = PagedWithStateSpec(PagedKVSpec(2, 40, 11, planes=1, keep_first=3), SlotStateSpec((30,)))
    other = PagedKVSpec(2, 40, 11, planes=1, keep_first=4)
    c = PagedCache([both, SlotStateSpec((7,)), both, other], [None] * 4, 8, 10, 3, 64, torch.float32, "cpu")
    assert c.group_entries == [2, 1] and sorted(c.states) == [0, 1, 2]
    b = c.binding(2)
    assert b.k.shape == (11, 2, 8, 40) and b.v is None and b.state.shape == (4, 30) and b.group == 0
    assert c.binding(3).state is None and c.binding(1).state.shape == (4, 7)
    assert c.manager.group(0).keep_first == 3 and c.manager.group(1).keep_first == 4
    assert PagedCache.bytes_per_token([both, SlotStateSpec((7,)), both, other], [None] * 4, torch.float32) == 3 * 2 * 40 * 4


# --------------------------------------------------------------------------- the plain restatement against second formulations

def test_plain_mask_and_softmax():
    m = S.visible(40, 7, 3)
    for i in range(40):
        for j in range(40):
            assert m[i, j] == (j <= i and (i - j < 7 or j < 3))
    assert S.visible(9, 100, 0).sum() == 45
    s = np.random.default_rng(0).normal(size=(5, 5)) * 3
    p = S.one_more_softmax(s, np.tril(np.ones((5, 5), dtype=bool)))
    for i in range(5):
        e = np.exp(s[i, :i + 1])
        assert np.allclose(p[i, :i + 1], e / (1 + e.sum())) and np.all(p[i, i + 1:] == 0)


def test_plain_convolution_is_causal_and_ends_on_the_token():
    u = np.random.default_rng(1).normal(size=(9, 2))
    w = np.array([[0.0, 0.0, 1.0], [2.0, 0.0, 0.0]])
    y = S.short_conv(u, w)
    assert np.allclose(y[:, 0], u[:, 0])
    assert np.allclose(y[2:, 1], 2 * u[:-2, 1]) and np.all(y[:2, 1] == 0)


def test_plain_delta_rule_is_the_error_correcting_write():
    """With decay 1 and beta 1 the state answers the key it has just been given with exactly that value."""
    rng = np.random.default_rng(2)
    D, Dv = 6, 4
    S_ = rng.normal(size=(D, Dv))
    k = rng.normal(size=D)
    k /= np.linalg.norm(k)
    v = rng.normal(size=Dv)
    S2 = S_ + np.outer(k, v - S_.T @ k)
    assert np.allclose(S2.T @ k, v)


def test_plain_router_chooses_by_corrected_scores_and_weighs_by_plain_ones():
    rng = np.random.default_rng(3)
    h = rng.normal(size=(50, 8))
    w = {"router": rng.normal(size=(6, 8)), "correction": np.array([0, 0, 5.0, 0, 0, 0])}
    idx, wts = S.route(h, w, "", {"experts": 4, "identity": 2, "top": 2, "scale": 1.5})
    assert np.all(idx[:, 0] == 2), "a large correction makes expert 2 every token's first choice"
    assert np.allclose(wts.sum(axis=1), 1.5)
    z = h @ w["router"].T
    s = np.exp(z) / np.exp(z).sum(axis=1, keepdims=True)
    t = 7
    assert np.allclose(wts[t, 0], 1.5 * s[t, 2] / (s[t, 2] + s[t, idx[t, 1]]))


def test_plain_identity_experts_hand_the_input_on():
    rng = np.random.default_rng(4)
    h = rng.normal(size=(5, 8))
    w = {"router": np.zeros((2, 8)), "correction": np.array([0.0, 1.0]), "e0.up": rng.normal(size=(3, 8)),
         "e0.down": rng.normal(size=(8, 3))}
    mlp = {"router": {"experts": 1, "identity": 1, "top": 1, "scale": 2.0}, "expert": {"ff": 3}}
    assert np.allclose(S.moe_ff(h, w, "", mlp), 2.0 * h)


def test_plain_forward_runs_the_passes():
    cfg = tiny.config([tiny.delta(heads=1, kv_heads=1, dim=4, vdim=4, conv=2)], width=8, vocab=11,
                      loop={"start": 0, "stop": 1, "times": 3})
    w = {k: v.float().numpy().astype(np.float64) for k, v in tiny.draw_weights(cfg, 0).items()}
    logits, layers = S.forward(cfg, w, [1, 2, 3], return_layers=True)
    assert layers.shape == (3, 3, 8) and logits.shape == (3, 11)
    # the second pass starts from the first pass's stream plus the embedding's output plus its own vector
    x0 = S.rms_norm(w["embed"][[1, 2, 3]], w["embed.norm"], 1e-5)
    x = layers[0] + x0 + w["loop.step"][1]
    h = S.rms_norm(x, w["l0.norm1"], 1e-5)
    assert np.allclose(layers[1], x + S.delta_mixer(h, w, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5))
