"""Venarax on the host: configuration, the model as data, what the cache manager makes of it, and the plain
implementation's own mechanisms."""
import copy

import numpy as np
import pytest

from machserve_b200.cache import CacheManager
from machserve_b200.config import ConfigError, config_from_json
from machserve_b200.parts import DecoderModel, PagedCache
from tests.plain import venarax as plain
from tests.venarax_cases import CASES


@pytest.mark.parametrize("name", sorted(CASES))
def test_config_round_trip_and_tensors(name):
    raw = CASES[name]["config"]
    cfg = config_from_json(raw)
    assert type(cfg).from_json(cfg.to_json()) == cfg
    model = DecoderModel(cfg.model_spec())
    decl = {d.name: tuple(d.shape) for d in model.tensors()}
    w = raw["width"]
    assert decl["embed"] == (raw["vocab"], w) and decl["head"] == (raw["vocab"], w)
    assert decl["final.norm"] == (w,) and decl["final.norm.b"] == (w,)
    for i, layer in enumerate(raw["layers"]):
        m, p = layer["mixer"], f"l{i}."
        assert decl[p + "norm1"] == (w,) and decl[p + "norm1.b"] == (w,)
        if layer["type"] == "attention":
            assert decl[p + "mix.q"] == (m["heads"] * m["dim"], w) and decl[p + "mix.k"] == (m["kv_heads"] * m["dim"], w)
            assert decl[p + "mix.v"] == (m["kv_heads"] * m["vdim"], w) and decl[p + "mix.o"] == (w, m["heads"] * m["vdim"])
            assert decl[p + "mix.q.norm"] == (m["heads"] * m["dim"],) and decl[p + "mix.sink"] == (m["heads"],)
        else:
            assert decl[p + "mix.q"] == (m["heads"] * (m["dim"] + m["rot_dim"]), w)
            assert decl[p + "mix.dkv"] == (m["kv_rank"] + m["rot_dim"], w) and decl[p + "mix.dkv.norm"] == (m["kv_rank"],)
            assert decl[p + "mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"]) and decl[p + "mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
            assert decl[p + "mix.g"] == (m["heads"] * m["vdim"], w) and decl[p + "mix.o"] == (w, m["heads"] * m["vdim"])
        if layer["mlp"] is None:
            assert p + "norm2" not in decl and p + "mlp.gate" not in decl
        else:
            assert decl[p + "mlp.gate"] == (layer["mlp"]["ff"], w) and decl[p + "mlp.down"] == (w, layer["mlp"]["ff"])
    assert ("loop.in" in decl) == ("loop" in raw)
    if "loop" in raw:
        assert decl["loop.in"] == (w, 2 * w) and decl["loop.step"] == (raw["loop"]["times"], w)


def test_run_order_follows_the_loop():
    cfg = config_from_json(CASES["P"]["config"])
    runs = cfg.model_spec().run_order
    assert [r.layer for r in runs] == [0, 1, 2, 1, 2, 3]
    assert [r.entry is not None for r in runs] == [False, True, False, True, False, False]
    assert [r.entry["row"] for r in runs if r.entry is not None] == [0, 1]
    assert all(r.cache_of is None for r in runs), "every pass has a cache of its own"
    assert [(i, t) for i, t in plain.run_order(CASES["P"]["config"])] == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (3, None)]
    none = config_from_json(CASES["Q"]["config"]).model_spec().run_order
    assert [r.layer for r in none] == [0, 1, 2, 3] and not any(r.entry for r in none)


def test_cache_groups_and_windows():
    cfg = config_from_json(CASES["S"]["config"])
    model = DecoderModel(cfg.model_spec())
    needs = model.cache_needs()
    assert len(needs) == 7 and all(isinstance(n, PagedCache) for n in needs)
    cache = CacheManager(needs, page_size=8, num_pages=12, num_state_slots=2)
    by_window = {g.need.window: g for g in cache.groups}
    assert set(by_window) == {None, 20}
    assert [p.name for p in by_window[20].need.planes] == ["latent"] and by_window[20].need.planes[0].width == 24 + 8
    assert len(by_window[20].runs) == 3, "the three passes of the looped latent layer are three runs of one group"
    # a request that grows token by token: the windowed group gives pages back, the other does not
    cache.begin("a")
    for n in range(1, 90):
        cache.reserve("a", n)
        cache.commit("a", n)
        cache.check()
    assert by_window[None].pool.num_held == 12 and by_window[20].pool.num_held <= 4
    cache.release("a")
    assert all(g.pool.num_held == 0 for g in cache.groups)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "not a mixer"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "experts"), "not supported"),
    (lambda c: c["loop"].__setitem__("stop", 9), "range"),
    (lambda c: c.pop("width"), "'width' is required"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "'scale' is required"),
])
def test_config_errors_name_the_key(change, message):
    raw = copy.deepcopy(CASES["P"]["config"])
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_json(raw)


# ------------------------------------------------------------------ the plain implementation's mechanisms


def test_plain_sink_takes_weight_and_has_no_value():
    rng = np.random.default_rng(0)
    s, v = rng.normal(size=(5, 5)), rng.normal(size=(5, 3))
    vis = plain.causal_mask(5)
    without = plain.softmax_attend(s, v, vis)
    assert np.allclose(plain.softmax_attend(s, v, vis, sink=-80.0), without)
    halved = plain.softmax_attend(s, v, vis, sink=float(np.log(np.exp(s[0, 0]))))
    assert np.allclose(halved[0], without[0] / 2), "a sink equal to the only score halves the row"


def test_plain_window_and_temperature_and_rotation():
    vis = plain.causal_mask(6, window=3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist() == [True, True, False, False, False, False]
    t = plain.query_temperature([0, 6, 7, 13, 14], 0.5, 7)
    assert np.allclose(t, [1, 1.0 + 0.5 * np.log(2), 1.0 + 0.5 * np.log(2), 1.0 + 0.5 * np.log(3), 1.0 + 0.5 * np.log(3)])
    x = np.arange(12, dtype=np.float64).reshape(1, 1, 12) + 1
    y = plain.rotate_pairs(x, [3], 100.0, 4)
    assert np.allclose(y[0, 0, 4:], x[0, 0, 4:]), "coordinates past the rotated ones pass unchanged"
    a = 3 * 100.0 ** (-2.0 * 1 / 4)
    assert np.allclose(y[0, 0, 2:4], [3 * np.cos(a) - 4 * np.sin(a), 4 * np.cos(a) + 3 * np.sin(a)])
    assert np.allclose(np.linalg.norm(y[0, 0, :4]), np.linalg.norm(x[0, 0, :4]))


def test_plain_clamps():
    w = {"gate": np.eye(3), "up": np.eye(3), "down": np.eye(3)}
    h = np.array([[5.0, -5.0, 0.5]])
    g, u = np.array([2.0, -5.0, 0.5]), np.array([2.0, -2.0, 0.5])
    want = g / (1 + np.exp(-1.702 * g)) * (u + 1)
    assert np.allclose(plain.clamped_gated_mlp(h, w, "", 2.0), want), "the gate is clamped from above only"
