"""Fozutar on the host: configuration, sizes that only the tensors give, the model as data, what the cache manager makes of
it, and the plain implementation's own mechanisms."""
import copy
import json

import numpy as np
import pytest

from machserve_b200.cache import CacheManager
from machserve_b200.config import ConfigError, config_from_json, load_config
from machserve_b200.parts import DecoderModel, FixedState, PagedCache
from machserve_b200.parts.chunked_attention import bias_by_distance, distance_bucket
from tests.fozutar_cases import CASES, make_model_dir
from tests.plain import fozutar as plain


@pytest.mark.parametrize("name", sorted(CASES))
def test_config_round_trip_and_tensors(name):
    raw = CASES[name]["config"]
    cfg = config_from_json(raw)
    assert type(cfg).from_json(cfg.to_json()) == cfg
    model = DecoderModel(cfg.model_spec())
    decl = {d.name: (tuple(d.shape), d.required) for d in model.tensors()}
    w = raw["width"]
    assert decl["embed"] == ((raw["vocab"], w), True) and decl["pos"] == ((raw["max_positions"], w), True)
    assert decl["head"][1] is False, "the head is the embedding table: a tensor of its own is optional"
    assert decl["final.norm"][0] == (w,)
    for i, layer in enumerate(raw["layers"]):
        m, p = layer["mixer"], f"l{i}."
        assert decl[p + "norm1"][0] == (w,) and p + "norm2" not in decl
        if layer["type"] == "attention":
            assert decl[p + "mix.q"][0] == (m["heads"] * m["dim"], w) and decl[p + "mix.k"][0] == (m["kv_heads"] * m["dim"], w)
            assert decl[p + "mix.q.b"][0] == (m["heads"] * m["dim"],) and decl[p + "mix.k.b"][0] == (m["kv_heads"] * m["dim"],)
            assert p + "mix.v" not in decl, "the values are the keys"
            assert decl[p + "mix.rel"][0] == (m["bias_rows"], m["heads"]) and decl[p + "mix.o"][0] == (w, m["heads"] * m["dim"])
        else:
            assert decl[p + "mix.q"][0] == (m["heads"] * m["dim"], w) and decl[p + "mix.v"][0] == (m["heads"] * m["vdim"], w)
            assert decl[p + "mix.a1"][0] == (m["decay_rank"], w) and decl[p + "mix.a2"][0] == (m["heads"] * m["dim"], m["decay_rank"])
            assert decl[p + "mix.a2.b"][0] == (m["heads"] * m["dim"],) and decl[p + "mix.norm"][0] == (m["vdim"],)
            assert decl[p + "mix.g"][0] == (m["heads"] * m["vdim"], w) and decl[p + "mix.o"][0] == (w, m["heads"] * m["vdim"])
        mlp = layer["mlp"]
        if mlp is None:
            assert not any(k.startswith(p + "mlp.") for k in decl)
        elif mlp["kind"] == "dense":
            assert decl[p + "mlp.gate"][0] == (mlp["ff"], w) and decl[p + "mlp.down"][0] == (w, mlp["ff"])
        else:
            e = mlp["router"]["experts"]
            assert decl[p + "mlp.router"][0] == (e, w) and decl[p + "mlp.router.b"][0] == (e,)
            assert decl[f"{p}mlp.e{e - 1}.up"][0] == (mlp["expert"]["ff"], w) and f"{p}mlp.e{e}.up" not in decl
    assert ("loop.step" in decl) == ("loop" in raw)
    if "loop" in raw:
        assert decl["loop.step"][0] == (raw["loop"]["times"], w)


def test_sizes_that_only_the_tensors_give(tmp_path):
    """config.json without the bias table's rows and the decay's rank: the folder's tensors say them."""
    d = make_model_dir(tmp_path, "A")
    raw = json.loads((d / "config.json").read_text())
    full = load_config(d)
    for layer in raw["layers"]:
        layer["mixer"].pop("bias_rows", None)
        layer["mixer"].pop("decay_rank", None)
    (d / "config.json").write_text(json.dumps(raw))
    bare = config_from_json(raw)
    assert bare.needs_tensor_shapes()
    with pytest.raises(ConfigError, match="only the tensors give"):
        bare.model_spec()
    assert load_config(d) == full


def test_optional_keys_of_the_attention():
    raw = copy.deepcopy(CASES["A"]["config"])
    m = raw["layers"][1]["mixer"]
    for key in ("softcap", "mask", "kv_heads"):
        m.pop(key)
    cfg = config_from_json(raw)
    a = cfg.layers[1].mixer
    assert a.softcap is None and a.chunk is None and a.kv_heads == a.heads
    assert type(cfg).from_json(cfg.to_json()) == cfg
    spec = cfg.model_spec().layers[1].mixer
    assert spec["softcap"] is None and spec["chunk"] is None
    need = DecoderModel(cfg.model_spec()).cache_needs()[1]
    assert need.chunk is None and need.window is None


def test_run_order_follows_the_loop():
    cfg = config_from_json(CASES["A"]["config"])
    runs = cfg.model_spec().run_order
    assert [r.layer for r in runs] == [0, 1, 2, 1, 2, 3]
    assert [r.entry is not None for r in runs] == [False, True, False, True, False, False]
    assert [(r.entry["row"], r.entry["add_first"]) for r in runs if r.entry is not None] == [(0, False), (1, True)]
    assert all(r.cache_of is None for r in runs), "every pass has a cache or state of its own"
    assert plain.run_order(CASES["A"]["config"]) == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (3, None)]
    none = config_from_json(CASES["B"]["config"]).model_spec().run_order
    assert [r.layer for r in none] == [0, 1, 2, 3] and not any(r.entry for r in none)


def test_cache_groups_states_and_chunks():
    cfg = config_from_json(CASES["D"]["config"])
    model = DecoderModel(cfg.model_spec())
    needs = model.cache_needs()
    assert len(needs) == 7
    assert [type(n) for n in needs] == [FixedState, PagedCache] * 3 + [PagedCache]
    assert needs[0].shape == (2, 12, 20)
    cache = CacheManager(needs, page_size=8, num_pages=12, num_state_slots=2)
    assert sorted(cache.state_runs) == [0, 2, 4], "each pass of the looped recurrent layer has a state of its own"
    by_chunk = {g.need.chunk: g for g in cache.groups}
    assert set(by_chunk) == {33, 48} and len(by_chunk[33].runs) == 3
    # a request that grows token by token holds the pages of its present chunk only
    cache.begin("a")
    for n in range(1, 90):
        cache.reserve("a", n)
        cache.commit("a", n)
        cache.check()
        for chunk, g in by_chunk.items():
            first = n // chunk * chunk  # the chunk of the next token
            assert g.pool.num_held <= (n - first) // 8 + 2
    cache.release("a")
    assert all(g.pool.num_held == 0 for g in cache.groups)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "not a mixer"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("vdim", 24), "values are the keys"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "experts"), "not supported"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "more than"),
    (lambda c: c["loop"].__setitem__("stop", 9), "range"),
    (lambda c: c.pop("width"), "'width' is required"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "'scale' is required"),
    (lambda c: c["layers"][0]["mixer"].pop("tau"), "'tau' is required"),
])
def test_config_errors_name_the_key(change, message):
    raw = copy.deepcopy(CASES["A"]["config"])
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_json(raw)


# ------------------------------------------------------------------ the mechanisms on the host


def test_distance_rows():
    # 8 rows that reach 40: distances 0..3 have rows of their own, then ln(n / 4) / ln(10) * 4 more
    got = [distance_bucket(n, 8, 40) for n in (0, 3, 4, 7, 8, 13, 22, 39, 40, 500)]
    assert got == [0, 3, 4, 4, 5, 6, 6, 7, 7, 7]
    assert [plain.distance_row(n, 8, 40) for n in range(60)] == [distance_bucket(n, 8, 40) for n in range(60)]
    import torch

    table = torch.arange(16, dtype=torch.float32).reshape(8, 2)
    by = bias_by_distance(table, 40, 50)
    assert by.shape == (2, 50) and by[1, 13].item() == table[6, 1].item() and by[0, 49].item() == table[7, 0].item()


def test_plain_chunks_and_cap():
    vis = plain.chunk_mask(7, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True, False]
    assert vis[3].tolist() == [False, False, False, True, False, False, False], "the first token of a chunk sees itself only"
    assert vis[2].tolist() == [True, True, True, False, False, False, False]
    assert plain.chunk_mask(4, None)[3].all()
    assert np.allclose(plain.soft_cap(np.array([0.01, 100.0, -100.0]), 5.0), [0.01, 5.0, -5.0], atol=1e-6)


def test_plain_recurrence_carries_its_state():
    rng = np.random.default_rng(0)
    q, k, g, v = rng.normal(size=(9, 4)), rng.normal(size=(9, 4)), -rng.uniform(0.01, 1.0, size=(9, 4)), rng.normal(size=(9, 3))
    whole, s_whole = plain.gla_recurrence(q, k, v, g)
    a, s = plain.gla_recurrence(q[:5], k[:5], v[:5], g[:5])
    b, s = plain.gla_recurrence(q[5:], k[5:], v[5:], g[5:], s)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(s, s_whole)
    # written out: o_t = sum_{s <= t} (q_t * prod_{s < r <= t} a_r) . k_s  v_s
    t = 6
    want = sum(((q[t] * np.exp(g[s0 + 1 : t + 1].sum(0))) @ k[s0]) * v[s0] for s0 in range(t + 1))
    assert np.allclose(whole[t], want)


def test_plain_router_takes_the_largest():
    w = {"router": np.eye(4), "router.b": np.array([0.0, 0.0, 0.5, 0.0])}
    ids, weights = plain.route(np.array([[0.1, 0.9, 0.3, -1.0]]), w, "", 2)
    assert ids.tolist() == [[1, 2]]
    e = np.exp([0.9, 0.8])
    assert np.allclose(weights[0], e / e.sum()), "the softmax is over the chosen logits only"


def test_a_library_of_some_of_the_kernel_files(tmp_path, monkeypatch):
    """A model whose parts name their kernel files is built a library of those files alone (when the whole library is not
    there): here the smallest such library, by the compiler, without a GPU."""
    import ctypes
    import shutil

    from machserve_b200.csrc import build

    if shutil.which("nvcc") is None and not (build.Path("/usr/local/cuda/bin/nvcc")).is_file():
        pytest.skip("no nvcc")
    cfg = config_from_json(CASES["A"]["config"])
    files = DecoderModel(cfg.model_spec()).kernel_files()
    assert files == ["attention_wide", "attention_wide_mma", "gla", "head_norm_store", "moe", "moe_grouped", "stream"]
    fp = build._fingerprint()
    monkeypatch.setattr(build, "_fingerprint", lambda flavor=None: fp + "x")  # as if no current library were anywhere
    monkeypatch.setenv("MACHSERVE_B200_BUILD_DIR", str(tmp_path))
    lib = build.library_for(["elementwise", "stream"], verbose=False)
    assert lib.parent == tmp_path and lib.name != build.LIB_NAME
    loaded = ctypes.CDLL(str(lib))
    assert hasattr(loaded, "ms_gated_act_mul") and hasattr(loaded, "ms_last_error") and not hasattr(loaded, "ms_gla_scan")
    assert build.library_for(["stream", "elementwise"], verbose=False) == lib, "the same files: the same library, not built again"
    with pytest.raises(build.BuildError, match="no such kernel files"):
        build.library_for(["no_such_file"], verbose=False)
