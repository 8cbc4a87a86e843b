"""Venarax on the GPU against the plain implementation: each mechanism's kernel alone, then the model in every way of
cutting the work (whole, token by token, portions down to two tokens, unequal requests side by side on reused pages),
and greedy generation through the engine."""
import json
import sys

import numpy as np
import pytest

from tests.helpers import (BF16_TOL, F32_TOL, REPO, assert_close, collect_rows, random_tokens, trace_portions, trace_tail_decode,
                           trace_whole)
from tests.plain import venarax as plain
from tests.venarax_cases import CASES, make_model_dir, plain_logits, read_weights

pytestmark = pytest.mark.gpu

MODEL_CASES = [(n, d) for n in sorted(CASES) for d in ("float32", "bfloat16")]


def _tol(dtype):
    return F32_TOL if dtype == "float32" else BF16_TOL


def _torch():
    import torch

    return torch


def _dev(a, dtype=None):
    torch = _torch()
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


# ----------------------------------------------------------------------------------- mechanisms, one kernel each


@pytest.mark.parametrize("d", [24, 50, 64, 200, 1000, 1531])
def test_layer_norm_adds_two_deltas_and_writes_two_norms(d):
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(d)
    x, a, b = (rng.normal(size=(9, d)).astype(np.float32) * s for s in (3.0, 1.0, 0.5))
    x += 2.0  # a mean that a norm without centring would get wrong
    w1, b1, w2, b2 = (rng.normal(size=d).astype(np.float32) for _ in range(4))
    res, out1, out2 = _dev(x), torch.empty(9, d, device="cuda"), torch.empty(9, d, device="cuda")
    ops.add_layernorm(res, _dev(a), _dev(b, torch.bfloat16), _dev(w1), _dev(b1), out1, 1e-5, None, _dev(w2), _dev(b2), out2)
    b_rounded = _dev(b, torch.bfloat16).float().cpu().numpy()
    s = x.astype(np.float64) + (a.astype(np.float64) + b_rounded)
    assert_close(res.cpu().numpy(), s, 1e-6, "stream after the add")
    assert_close(out1.cpu().numpy(), plain.layer_norm(s, w1, b1, 1e-5), 2e-5, "first norm")
    assert_close(out2.cpu().numpy(), plain.layer_norm(s, w2, b2, 1e-5), 2e-5, "second norm")
    # picked rows: nothing is written back
    rows = torch.tensor([7, 0, 7], dtype=torch.int32, device="cuda")
    res2, picked = _dev(x), torch.empty(3, d, device="cuda")
    ops.add_layernorm(res2, _dev(a), None, _dev(w1), _dev(b1), picked, 1e-5, rows)
    assert np.array_equal(res2.cpu().numpy(), x)
    assert_close(picked.cpu().numpy(), plain.layer_norm((x.astype(np.float64) + a)[[7, 0, 7]], w1, b1, 1e-5), 2e-5, "picked rows")


def test_clamped_gated_unit_and_sigmoid_gate():
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(1)
    gu = (rng.normal(size=(5, 2 * 37)) * 3).astype(np.float32)
    for limit in (0.7, 2.0):
        out = torch.empty(5, 37, device="cuda")
        ops.glu_clamped(_dev(gu), out, limit, 1.702, 1.0)
        eye = {"gate": np.eye(37), "up": np.eye(37), "down": np.eye(37)}
        g = np.minimum(gu[:, :37].astype(np.float64), limit)
        u = np.clip(gu[:, 37:].astype(np.float64), -limit, limit)
        assert_close(out.cpu().numpy(), g / (1 + np.exp(-1.702 * g)) * (u + 1), 1e-6, f"limit {limit}")
        assert (gu[:, :37] < -limit).any() and (gu[:, :37] > limit).any(), "the test's gates reach past both limits"
    x, gate = rng.normal(size=(4, 50)).astype(np.float32), rng.normal(size=(4, 90)).astype(np.float32) * 4
    out = torch.empty(4, 50, device="cuda")
    ops.sigmoid_gate_mul(_dev(x), _dev(gate)[:, 40:], out)
    assert_close(out.cpu().numpy(), x / (1 + np.exp(-gate[:, 40:].astype(np.float64))), 1e-6, "sigmoid gate on a column range")


def _paged(rng, tokens_per_seq, heads, width, page, dtype, spare=3):
    """Pages in shuffled order for sequences of the given lengths: (pages array, block table, host copy by sequence)."""
    torch = _torch()
    per = [-(-n // page) for n in tokens_per_seq]
    ids = rng.permutation(sum(per) + spare)
    table = np.full((len(per), max(per) + 1), -1, dtype=np.int32)
    pages = np.zeros((sum(per) + spare, heads, page, width), dtype=np.float32)
    at = 0
    for s, n in enumerate(per):
        table[s, :n] = ids[at : at + n]
        at += n
    return pages, table


def _fill_pages(pages, table, seq, values, page):
    """values [tokens, heads, width] of sequence `seq` into its pages."""
    for p in range(values.shape[0]):
        pages[table[seq, p // page], :, p % page, :] = values[p]


def _plain_attend(q, k, v, positions, window, scale, sinks, groups):
    """q [T, H, dk] at `positions` of one sequence whose keys k [N, G, dk] and values v [N, G, dv] are all there."""
    t, h, _ = q.shape
    out = np.zeros((t, h, v.shape[2]))
    for i, p in enumerate(positions):
        lo = 0 if not window else max(0, p - window + 1)
        vis = np.zeros((1, k.shape[0]), dtype=bool)
        vis[0, lo : p + 1] = True
        for head in range(h):
            g = head // groups
            s = (q[i, head][None, :] @ k[:, g].T) * scale
            out[i, head] = plain.softmax_attend(s, v[:, g], vis, None if sinks is None else float(sinks[head]))[0]
    return out


@pytest.mark.parametrize("dk,dv,hq,hkv,window,sink,page", [
    (24, 16, 4, 2, None, True, 8), (7, 20, 6, 1, None, True, 16), (40, 40, 2, 2, 19, False, 8), (152, 136, 3, 1, 33, False, 16),
    (16, 144, 2, 1, None, True, 16), (20, 300, 2, 2, 50, True, 8), (96, 96, 8, 2, None, True, 16),
])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_with_sink_and_unequal_widths(dk, dv, hq, hkv, window, sink, page, dtype):
    """Portions of two sequences side by side and decoded rows, against the plain softmax; the two forms of the kernel
    (rows of a portion share a block; heads of a token share a block) give the same bits."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(dk * 1000 + dv)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    lens = [75, 41]
    kp, table = _paged(rng, lens, hkv, dk, page, dtype)
    vp = np.zeros(kp.shape[:3] + (dv,), dtype=np.float32)
    ks = [rng.normal(size=(n, hkv, dk)).astype(np.float32) for n in lens]
    vs = [rng.normal(size=(n, hkv, dv)).astype(np.float32) for n in lens]
    for s in range(2):
        _fill_pages(kp, table, s, ks[s], page)
        _fill_pages(vp, table, s, vs[s], page)
    kd, vd = _dev(kp, tdt), _dev(vp, tdt)
    ks = [_dev(k, tdt).float().cpu().numpy().astype(np.float64) for k in ks]  # what the cache holds
    vs = [_dev(v, tdt).float().cpu().numpy().astype(np.float64) for v in vs]
    sinks = rng.normal(size=hq).astype(np.float32) * 2 if sink else None
    scale = 0.4 / np.sqrt(dk)
    # rows: the last 30 positions of sequence 0 (a portion), the last position of sequence 1 (a decoded row), then the
    # first three positions of sequence 1 as a short portion
    rows = [(0, p) for p in range(45, 75)] + [(1, 40)] + [(1, p) for p in range(3)]
    q = rng.normal(size=(len(rows), hq, dk)).astype(np.float32)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device="cuda")
    slot = torch.tensor([s for s, _ in rows], dtype=torch.int32, device="cuda")
    outs = []
    for share in (True, False):
        out = torch.zeros(len(rows), hq * dv, dtype=tdt, device="cuda")
        ops.attention_wide(_dev(q).view(len(rows), hq * dk), kd, vd, out, None if sinks is None else _dev(sinks), pos, slot, _dev(table),
                           hq, hkv, dk, dv, window, scale, share_rows=share)
        outs.append(out.float().cpu().numpy().reshape(len(rows), hq, dv))
    assert np.array_equal(outs[0], outs[1]), "rows that share a block and heads that share a block must give the same bits"
    want = np.zeros((len(rows), hq, dv))
    for s in range(2):
        idx = [i for i, (ss, _) in enumerate(rows) if ss == s]
        want[idx] = _plain_attend(q[idx].astype(np.float64), ks[s], vs[s], [rows[i][1] for i in idx], window, scale, sinks, hq // hkv)
    assert_close(outs[0].reshape(len(rows), -1), want.reshape(len(rows), -1), 2e-5 if dtype == "float32" else 1e-2, "attention")


@pytest.mark.parametrize("dk,dv,hq,hkv,window,sink,latent,page", [
    (64, 64, 4, 2, None, True, False, 16), (96, 96, 6, 2, None, True, False, 8), (48, 80, 3, 1, 21, True, False, 16),
    (160, 128, 4, 1, 33, False, True, 16), (288, 256, 14, 1, 50, False, True, 16), (576, 512, 2, 1, 40, False, True, 8),
    (32, 24, 20, 1, None, True, False, 8),
])
def test_tensor_core_attention_with_sink_and_unequal_widths(dk, dv, hq, hkv, window, sink, latent, page):
    """The bfloat16 tensor-core form: tiles of rows of two sequences, decoding rows whose keys are cut into runs that
    are merged, values inside the keys' own plane (a latent cache), against the plain softmax and the exact kernel."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(dk * 7 + dv)
    bf = torch.bfloat16
    lens = [150, 41]
    kp, table = _paged(rng, lens, hkv, dk, page, "bfloat16")
    ks = [rng.normal(size=(n, hkv, dk)).astype(np.float32) for n in lens]
    for s in range(2):
        _fill_pages(kp, table, s, ks[s], page)
    kd = _dev(kp, bf)
    if latent:
        vd, vs = kd, [k[:, :, :dv] for k in ks]
    else:
        vp = np.zeros(kp.shape[:3] + (dv,), dtype=np.float32)
        vs = [rng.normal(size=(n, hkv, dv)).astype(np.float32) for n in lens]
        for s in range(2):
            _fill_pages(vp, table, s, vs[s], page)
        vd = _dev(vp, bf)
    ks = [_dev(k, bf).float().cpu().numpy().astype(np.float64) for k in ks]
    vs = [_dev(np.ascontiguousarray(v), bf).float().cpu().numpy().astype(np.float64) for v in vs]
    assert ops.attention_wide_mma_supports(dk, dv, vd.shape[3], not latent)
    sinks = rng.normal(size=hq).astype(np.float32) * 2 if sink else None
    scale = 0.5 / np.sqrt(dk)
    # rows 0..36: positions 100..136 of sequence 0 (in tiles of as many rows as a block takes); row 37: the last position of sequence 0,
    # decoded; rows 38..40: the first three positions of sequence 1; row 41: position 40 of sequence 1, decoded
    rows = [(0, p) for p in range(100, 137)] + [(0, 149)] + [(1, p) for p in range(3)] + [(1, 40)]
    q = rng.normal(size=(len(rows), hq, dk)).astype(np.float32)
    q_held = _dev(q, bf).float().cpu().numpy().astype(np.float64)  # the tensor core reads the queries as bfloat16
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device="cuda")
    slot = torch.tensor([s for s, _ in rows], dtype=torch.int32, device="cuda")
    ints = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    want = np.zeros((len(rows), hq, dv))
    for s in range(2):
        idx = [i for i, (ss, _) in enumerate(rows) if ss == s]
        want[idx] = _plain_attend(q_held[idx], ks[s], vs[s], [rows[i][1] for i in idx], window, scale, sinks, hq // hkv)
    sk = None if sinks is None else _dev(sinks)
    tile = ops.attention_wide_mma_tile_rows(dv)
    assert tile == (64 if dv <= 128 else 32 if dv <= 256 else 16)
    t0 = list(range(0, 37, tile)) + [38, 0]
    tn = [min(tile, 37 - a) for a in range(0, 37, tile)] + [3, 0]
    for splits in (1, 3):
        out = torch.full((len(rows), hq * dv), 7.0, dtype=bf, device="cuda")
        ops.attention_wide_mma(_dev(q).view(len(rows), hq * dk), kd, vd, out, sk, pos, slot, _dev(table), ints(t0), ints(tn), len(t0), False,
                               hq, hkv, dk, dv, window, scale)
        items = 3 * hkv * (-(-(hq // hkv) // 16))
        scratch = torch.empty(max(1, ops.attention_wide_mma_scratch_words(items, dv, splits)), device="cuda")
        ops.attention_wide_mma(_dev(q).view(len(rows), hq * dk), kd, vd, out, sk, pos, slot, _dev(table), ints([37, -1, 41]), None, 3, True,
                               hq, hkv, dk, dv, window, scale, splits, scratch)
        assert_close(out.float().cpu().numpy(), want.reshape(len(rows), -1), 1.5e-2, f"tensor-core attention, {splits} runs of keys")
    exact = torch.zeros(len(rows), hq * dv, dtype=bf, device="cuda")
    ops.attention_wide(_dev(q).view(len(rows), hq * dk), kd, vd, exact, sk, pos, slot, _dev(table), hq, hkv, dk, dv, window, scale, share_rows=True)
    assert_close(out.float().cpu().numpy(), exact.float().cpu().numpy(), 2e-2, "tensor-core form against the exact kernel")


@pytest.mark.parametrize("hd,hq,hkv,n,splits", [(64, 4, 2, 300, 1), (64, 6, 1, 700, 3), (128, 4, 2, 300, 1), (128, 6, 2, 700, 2),
                                                  (128, 3, 1, 520, 4)])
def test_sink_in_the_tcgen05_attention(hd, hq, hkv, n, splits):
    """The framework's tcgen05 attention for prompt portions with a sink per head in its finish: one head a block (head
    size 64) and two heads of a group a block (128), whole and with the key tiles cut into runs that are merged; against
    the exact kernel with the same sinks, and without sinks against itself as it was."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(hd + n)
    bf, page = torch.bfloat16, 16
    kp, table = _paged(rng, [n], hkv, hd, page, "bfloat16")
    vp = np.zeros_like(kp)
    _fill_pages(kp, table, 0, rng.normal(size=(n, hkv, hd)).astype(np.float32), page)
    _fill_pages(vp, table, 0, rng.normal(size=(n, hkv, hd)).astype(np.float32), page)
    kd, vd = _dev(kp, bf), _dev(vp, bf)
    q = _dev(rng.normal(size=(n, hq * hd)).astype(np.float32), bf)
    sinks = _dev((rng.normal(size=hq) + np.log(n / 2)).astype(np.float32))  # about half of a middle row's weight
    pos = torch.arange(n, dtype=torch.int32, device="cuda")
    slot = torch.zeros(n, dtype=torch.int32, device="cuda")
    t0 = torch.arange(0, n, 128, dtype=torch.int32, device="cuda")
    tn = torch.tensor([min(128, n - a) for a in range(0, n, 128)], dtype=torch.int32, device="cuda")
    tiles, scale = t0.numel(), hd ** -0.5
    scratch = counters = None
    if splits > 1:
        scratch = torch.zeros(ops.attention_prefill_tc_scratch_words(tiles, hq, hd, splits), device="cuda")
        counters = torch.zeros(tiles * hq, dtype=torch.int32, device="cuda")
    outs = {}
    for name, sk in (("sinks", sinks), ("plain", None)):
        out = torch.zeros(n, hq * hd, dtype=bf, device="cuda")
        ops.attention_prefill_tc(q, kd, vd, out, t0, tn, tiles, pos, slot, _dev(table), hq, hkv, hd, None, scale, splits, scratch, counters,
                                 sinks=sk)
        exact = torch.zeros(n, hq * hd, dtype=bf, device="cuda")
        ops.attention_wide(q.float(), kd, vd, exact, sk, pos, slot, _dev(table), hq, hkv, hd, hd, None, scale, share_rows=True)
        assert_close(out.float().cpu().numpy(), exact.float().cpu().numpy(), 2e-2, f"tcgen05 attention, {name}, {splits} runs")
        outs[name] = out.float().cpu().numpy()
    assert ops.tc_status_codes() == (0, 0)
    if counters is not None:
        assert int(counters.abs().sum()) == 0, "the counters are left zero"
    assert np.abs(outs["sinks"] - outs["plain"]).max() > 0.05, "the test's sinks matter"


@pytest.mark.parametrize("hd,hq,hkv,rows,ctx", [(64, 4, 2, 5, 300), (96, 4, 2, 8, 1100), (128, 8, 2, 3, 700), (64, 14, 2, 2, 9000),
                                                  (128, 4, 1, 1, 6000), (32, 6, 3, 20, 150)])
def test_sink_in_the_cluster_decode_attention(hd, hq, hkv, rows, ctx):
    """The framework's decode kernel (clusters of blocks over a row's keys, several clusters a row for few rows with long
    contexts) with a sink per head in its merges, launched by its own rules; against the exact kernel with the same sinks."""
    torch = _torch()
    from types import SimpleNamespace

    from machserve_b200 import ops
    from machserve_b200.parts.attention import decode_launch

    rng = np.random.default_rng(hd + ctx)
    bf, page = torch.bfloat16, 16
    lens = [ctx - 7 * i for i in range(rows)]
    kp, table = _paged(rng, lens, hkv, hd, page, "bfloat16")
    kd = _dev(rng.normal(size=kp.shape).astype(np.float32), bf)
    vd = _dev(rng.normal(size=kp.shape).astype(np.float32), bf)
    q = _dev(rng.normal(size=(rows, hq * hd)).astype(np.float32), bf)
    sinks = _dev((rng.normal(size=hq) + np.log(ctx)).astype(np.float32))  # about half of a row's weight
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    slot = torch.arange(rows, dtype=torch.int32, device="cuda")
    scale = hd ** -0.5
    rt = SimpleNamespace(sm_count=torch.cuda.get_device_properties(0).multi_processor_count)
    splits, stages, warps, kpw, parts = decode_launch(rt, hd, ops.attention_decode_cluster_max_stages(hd), {}, rows * hkv, -(-ctx // 64))
    scratch = counters = None
    if parts > 1:
        scratch = torch.zeros(ops.attention_decode_cluster_scratch_words(rows, hq, hkv, hd, parts), device="cuda")
        counters = torch.zeros(rows * hkv, dtype=torch.int32, device="cuda")
    outs = {}
    for name, sk in (("sinks", sinks), ("plain", None)):
        out = torch.zeros(rows, hq * hd, dtype=bf, device="cuda")
        ops.attention_decode_cluster(q, kd, vd, out, pos, slot, _dev(table), hq, hkv, hd, None, scale, splits, stages, warps=warps,
                                     keys_per_warp=kpw, parts=parts, scratch=scratch, counters=counters, sinks=sk)
        exact = torch.zeros(rows, hq * hd, dtype=bf, device="cuda")
        ops.attention_wide(q.float(), kd, vd, exact, sk, pos, slot, _dev(table), hq, hkv, hd, hd, None, scale)
        assert_close(out.float().cpu().numpy(), exact.float().cpu().numpy(), 2e-2,
                     f"cluster decode, {name}, {splits} splits, {parts} clusters a row")
        outs[name] = out.float().cpu().numpy()
    if (hd, rows) in ((64, 2), (128, 1)):
        assert parts > 1, "the long contexts of few rows are meant to go to several clusters a row"
    assert np.abs(outs["sinks"] - outs["plain"]).max() > 0.02, "the test's sinks matter"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_one_key_stands_out(dtype):
    """One key among hundreds is made to carry nearly all the weight.  Far back, on a page border, just inside the
    window it must be found; just outside the window it must not be seen; a large sink must take the weight instead."""
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(5)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    dk, dv, page, n, window = 32, 48, 16, 700, 96
    kp, table = _paged(rng, [n], 1, dk, page, dtype)
    vp = np.zeros(kp.shape[:3] + (dv,), dtype=np.float32)
    k = rng.normal(size=(n, 1, dk)).astype(np.float32) * 0.1
    v = rng.normal(size=(n, 1, dv)).astype(np.float32)
    direction = rng.normal(size=dk).astype(np.float32)
    direction /= np.linalg.norm(direction)
    marked = {0: "first key", 15: "end of a page", 16: "start of a page", 300: "far", 699 - window: "just outside", 700 - window: "just inside"}
    for j in marked:
        k[j, 0] = 0  # they are switched on one at a time below
    _fill_pages(vp, table, 0, v, page)
    q = (direction * 40.0)[None, None, :].astype(np.float32)
    pos = torch.tensor([n - 1], dtype=torch.int32, device="cuda")
    slot = torch.zeros(1, dtype=torch.int32, device="cuda")
    vd = _dev(vp, tdt)
    v_held = vd.float().cpu().numpy()

    def attend(key_at, win, sinks=None):
        kk = k.copy()
        kk[key_at, 0] = direction  # score 40 against scores near 0
        kp2 = kp.copy()
        _fill_pages(kp2, table, 0, kk, page)
        out = torch.zeros(1, dv, dtype=tdt, device="cuda")
        ops.attention_wide(_dev(q).view(1, dk), _dev(kp2, tdt), vd, out, sinks, pos, slot, _dev(table), 1, 1, dk, dv, win, 1.0)
        return out.float().cpu().numpy()[0]

    tol = 1e-4 if dtype == "float32" else 5e-2
    for j, what in marked.items():
        found = v_held[table[0, j // page], 0, j % page]
        assert np.abs(attend(j, None) - found).max() < tol, f"without a window the key at {j} ({what}) carries the row"
        inside = j >= n - window
        got = attend(j, window)
        assert (np.abs(got - found).max() < tol) == inside, f"with a window of {window} the key at {j} ({what}) is {'seen' if inside else 'not seen'}"
    big = torch.tensor([60.0], device="cuda")
    assert np.abs(attend(603, None, big)).max() < 1e-6, "a sink far above every score takes the weight and has no value"
    level = torch.tensor([40.0], device="cuda")
    found = v_held[table[0, 603 // page], 0, 603 % page]
    assert np.abs(attend(603, None, level) - found / 2).max() < tol, "a sink level with the one score halves the row; it is not scaled"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_query_key_norm_temperature_and_store(dtype):
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(2)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    hq, g, dk, dv, page, every, coef, eps = 3, 1, 10, 6, 8, 4, 0.8, 1e-3
    qw, kw, vw = hq * dk, g * dk, g * dv
    positions = [0, 2, 3, 4, 11, 12, 30]
    proj = rng.normal(size=(len(positions), qw + kw + vw + 5)).astype(np.float32)  # a wider product: the rows have a stride
    wq, wk = rng.normal(size=qw).astype(np.float32), rng.normal(size=kw).astype(np.float32)
    kp, table = _paged(rng, [31], g, dk, page, dtype)
    k_pages, v_pages = torch.zeros(kp.shape, dtype=tdt, device="cuda"), torch.zeros(kp.shape[:3] + (dv,), dtype=tdt, device="cuda")
    q_out = torch.empty(len(positions), qw, device="cuda")
    ops.qk_norm_store(_dev(proj), _dev(wq), _dev(wk), eps, coef, every, torch.tensor(positions, dtype=torch.int32, device="cuda"),
                      torch.zeros(len(positions), dtype=torch.int32, device="cuda"), _dev(table), q_out, k_pages, v_pages, g, dk, dv)
    p64 = proj.astype(np.float64)
    want_q = plain.unit_rms(p64[:, :qw], eps) * wq * plain.query_temperature(positions, coef, every)[:, None]
    assert_close(q_out.cpu().numpy(), want_q, 2e-6, "queries")
    assert plain.query_temperature([2], coef, every)[0] == 1.0 and plain.query_temperature([3], coef, every)[0] > 1.0
    want_k = plain.unit_rms(p64[:, qw : qw + kw], eps) * wk
    tol = 2e-6 if dtype == "float32" else 1e-2
    for i, p in enumerate(positions):
        page_id = table[0, p // page]
        assert_close(k_pages[page_id, :, p % page].float().cpu().numpy().reshape(-1), want_k[i], tol, f"key at {p}")
        assert_close(v_pages[page_id, :, p % page].float().cpu().numpy().reshape(-1), p64[i, qw + kw : qw + kw + vw], tol, f"value at {p}")


@pytest.mark.parametrize("rot", [6, 2, 0])
def test_latent_encode(rot):
    torch = _torch()
    from machserve_b200 import ops

    rng = np.random.default_rng(rot)
    heads, dn, dr, r, page, base, eps = 3, 5, 6, 12, 8, 77.0, 1e-4
    positions = [0, 1, 7, 8, 20]
    qw = heads * (dn + dr)
    proj = rng.normal(size=(len(positions), qw + r + dr + 3)).astype(np.float32)
    w = rng.normal(size=r).astype(np.float32)
    i = np.arange(max(rot, 2) // 2, dtype=np.float64)
    ang = np.arange(32, dtype=np.float64)[:, None] * base ** (-2.0 * i / max(rot, 2))[None, :]
    table_cs = np.stack([np.cos(ang), np.sin(ang)], -1).astype(np.float32) if rot else None
    pg, table = _paged(rng, [21], 1, r + dr, page, "float32")
    pages = torch.zeros(pg.shape, device="cuda")
    q_wide = torch.zeros(len(positions), heads, r + dr, device="cuda")
    q_plain = torch.zeros(len(positions), heads, dn, device="cuda")
    ops.latent_encode(_dev(proj), qw, _dev(w), eps, None if table_cs is None else _dev(table_cs), rot,
                      torch.tensor(positions, dtype=torch.int32, device="cuda"), torch.zeros(len(positions), dtype=torch.int32, device="cuda"),
                      _dev(table), q_wide, q_plain, pages, heads, dn, dr, r)
    p64 = proj.astype(np.float64)
    q = p64[:, :qw].reshape(len(positions), heads, dn + dr)
    turned_q = plain.rotate_pairs(q[..., dn:], positions, base, rot) if rot else q[..., dn:]
    assert_close(q_plain.cpu().numpy().reshape(len(positions), -1), q[..., :dn].reshape(len(positions), -1), 1e-7, "unrotated query parts")
    assert_close(q_wide[:, :, r:].cpu().numpy().reshape(len(positions), -1), turned_q.reshape(len(positions), -1), 2e-6, "rotated query parts")
    c = plain.unit_rms(p64[:, qw : qw + r], eps) * w
    kr = p64[:, None, qw + r : qw + r + dr]
    kr = (plain.rotate_pairs(kr, positions, base, rot) if rot else kr)[:, 0]
    for n, p in enumerate(positions):
        got = pages[table[0, p // page], 0, p % page].cpu().numpy()
        assert_close(got, np.concatenate([c[n], kr[n]]), 2e-6, f"[latent | key part] at {p}")


# ----------------------------------------------------------------------------------- the model, cut every way


def _replay(model_dir, dtype, steps, max_tokens, page, max_requests=4):
    from machserve_b200.engine.replay import make_replay_runner, replay

    runner = make_replay_runner(model_dir, dtype, max_tokens, page, max_requests)
    out = replay(runner, steps)
    runner.cache.check()
    assert not runner.cache.requests, "requests still hold cache after the trace ended"
    assert all(g.pool.num_held == 0 for g in runner.cache.groups)
    return out


def _want(model_dir, dtype, tokens):
    return plain_logits(model_dir, tokens, bf16_weights=(dtype == "bfloat16"))


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_whole_prompts(model_root, name, dtype):
    """Each request alone and whole, every position wanted: the first tokens of a sequence are among them."""
    d = make_model_dir(model_root, name)
    requests = {f"r{n}": random_tokens(CASES[name]["config"]["vocab"], n, 300 + n) for n in (1, 2, 9, 33, 70)}
    steps = trace_whole(requests)
    got = collect_rows(steps, _replay(d, dtype, steps, 128, CASES[name]["page"]))
    for rid, toks in requests.items():
        assert_close(got[rid], _want(d, dtype, toks), _tol(dtype), f"{name} {dtype} whole {rid}")


@pytest.mark.parametrize("name", sorted(CASES))
def test_layers_follow_the_plain_layers(model_root, name):
    """The stream after every run of a layer (a looped layer counts each time) against the plain layers."""
    from machserve_b200.engine.replay import make_replay_runner
    from machserve_b200.engine.runner import StepEntry

    d = make_model_dir(model_root, name)
    toks = random_tokens(CASES[name]["config"]["vocab"], 37, 1)
    runner = make_replay_runner(d, "float32", 64, CASES[name]["page"])
    taps = []
    runner.step([StepEntry("a", toks, [0])], tap=lambda i, h: taps.append(h.cpu().numpy()) if i >= 0 else None)
    cfg, w = read_weights(d)
    want = []
    plain.forward(cfg, w, toks, want)
    assert len(taps) == len(want) == len(plain.run_order(cfg))
    for i, (a, b) in enumerate(zip(taps, want)):
        assert_close(a, b, F32_TOL, f"{name}: stream after run {i}")


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_decoded_tail_passes_every_window(model_root, name, dtype):
    """Most of it in one step, the last 48 tokens one by one: more than every window of the tiny models, so that
    decoded tokens leave the windows, and windows' edges fall among decoded tokens."""
    d = make_model_dir(model_root, name)
    toks = random_tokens(CASES[name]["config"]["vocab"], 90, 7)
    steps = trace_tail_decode("a", toks, 48)
    got = collect_rows(steps, _replay(d, dtype, steps, 128, CASES[name]["page"]))
    assert_close(got["a"], _want(d, dtype, toks), _tol(dtype), f"{name} {dtype} tail")


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_portions_down_to_two_tokens(model_root, name, dtype):
    d = make_model_dir(model_root, name)
    toks = random_tokens(CASES[name]["config"]["vocab"], 100, 11)
    steps = trace_portions("a", toks, [7, 2, 13, 3, 2, 16, 5, 9, 31])
    got = collect_rows(steps, _replay(d, dtype, steps, 128, CASES[name]["page"]))["a"]
    assert_close(got, _want(d, dtype, toks), _tol(dtype), f"{name} {dtype} portions")
    if dtype == "float32":  # the arithmetic of a row depends on its position alone
        whole = trace_whole({"a": toks})
        alone = collect_rows(whole, _replay(d, dtype, whole, 128, CASES[name]["page"]))["a"]
        assert np.array_equal(got, alone), "float32 logits must not depend on how the prompt was cut"


@pytest.mark.parametrize("name,dtype", MODEL_CASES)
def test_unequal_requests_side_by_side_on_reused_pages(model_root, name, dtype):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool so small that later
    requests run on pages and slots that earlier ones gave back; each against itself alone."""
    from tests.test_replay_gpu import mixed_trace

    d = make_model_dir(model_root, name)
    requests, steps = mixed_trace(CASES[name]["config"]["vocab"], seed=5)
    assert max(len(s["entries"]) for s in steps) >= 3
    got = collect_rows(steps, _replay(d, dtype, steps, 256, CASES[name]["page"], max_requests=4))
    for rid, toks in requests.items():
        assert_close(got[rid], _want(d, dtype, toks), _tol(dtype), f"{name} {dtype} mixed {rid}")
    if dtype == "float32":
        whole = trace_whole(requests)
        alone = collect_rows(whole, _replay(d, dtype, whole, 256, CASES[name]["page"]))
        for rid in requests:
            assert np.array_equal(got[rid], alone[rid]), f"float32 logits of {rid} must not depend on the batch or the pages"


@pytest.mark.parametrize("name,dtype", [("T", "bfloat16"), ("U", "bfloat16"), ("P", "float32")])
def test_many_rows_decode_together(model_root, name, dtype):
    """24 requests of unequal lengths decode side by side for several steps (more rows than the few-row products take,
    so the products go to the library), then half of them end and others go on: each against itself alone."""
    from machserve_b200.engine.replay import make_replay_runner, replay

    d = make_model_dir(model_root, name)
    vocab = CASES[name]["config"]["vocab"]
    lens = [5 + 3 * i for i in range(24)]
    reqs = {f"r{i}": random_tokens(vocab, n + 6, 500 + i) for i, n in enumerate(lens)}
    steps, st = [], 0
    for rid, toks in reqs.items():  # the prompts, one request a step
        steps.append({"step": st, "entries": [{"id": rid, "tokens": toks[:-6], "want": [len(toks) - 7]}], "end": []})
        st += 1
    for k in range(6):  # six decoding steps; after the third, the even requests are left out (they end early)
        live = [rid for i, rid in enumerate(reqs) if k < 3 or i % 2]
        ended = [rid for i, rid in enumerate(reqs) if (k == 2 and i % 2 == 0) or (k == 5 and i % 2)]
        steps.append({"step": st, "entries": [{"id": rid, "tokens": [reqs[rid][len(reqs[rid]) - 6 + k]], "want": [0]} for rid in live],
                      "end": ended})
        st += 1
    runner = make_replay_runner(d, dtype, 24 * 128, CASES[name]["page"], 24)
    got = collect_rows(steps, replay(runner, steps))
    runner.cache.check()
    assert not runner.cache.requests
    for i, (rid, toks) in enumerate(reqs.items()):
        n = len(toks) if i % 2 else len(toks) - 3
        want = _want(d, dtype, toks[:n])[len(toks) - 7 : n]
        assert_close(got[rid], want, _tol(dtype), f"{name} {dtype} {rid} among 24")


@pytest.mark.parametrize("name", ["P", "Q"])
def test_long_decoding(model_root, name):
    """Token by token from the first token on, far past every window and over many pages."""
    d = make_model_dir(model_root, name)
    toks = random_tokens(CASES[name]["config"]["vocab"], 150, 21)
    steps = trace_tail_decode("a", toks, 149)
    for dtype in ("float32", "bfloat16"):
        got = collect_rows(steps, _replay(d, dtype, steps, 192, CASES[name]["page"]))
        assert_close(got["a"], _want(d, dtype, toks), _tol(dtype), f"{name} {dtype} long decoding")


@pytest.mark.parametrize("name,dtype", [("Q", "float32"), ("U", "bfloat16"), ("T", "bfloat16")])
def test_a_large_sink_shows_in_the_logits(model_root, tmp_path, name, dtype):
    """The sinks of a model are raised until they take most of every head's weight: the engine follows the plain model
    (in bfloat16 through the tensor-core kernels: tcgen05 for the prompt at key rows of 64, mma.sync else)."""
    torch = _torch()
    from machserve_b200.config import load_config
    from machserve_b200.engine.runner import ModelRunner, StepEntry
    from machserve_b200.parts import DecoderModel
    from machserve_b200.weights import load_weights

    d = make_model_dir(model_root, name)
    config = load_config(d)
    tensors = load_weights(d, DecoderModel(config.model_spec()).tensors(), torch.float32, "cpu")
    cfg, w = read_weights(d, round_to_bf16=(dtype == "bfloat16"))
    toks = random_tokens(cfg["vocab"], 150, 3)
    before = plain.forward(cfg, w, toks)
    for name in tensors:
        if name.endswith("mix.sink"):
            tensors[name] = tensors[name] + 4.0
            w[name] = w[name] + 4.0
    after = plain.forward(cfg, w, toks)
    assert np.abs(after - before).max() > 0.05, "the test's sinks matter"
    runner = ModelRunner(config, tensors, dtype=dtype, page_size=16, num_pages=16, max_requests=2, max_step_tokens=256)
    got = runner.step([StepEntry("a", toks[:140], list(range(140)))]).cpu().numpy()
    assert_close(got, after[:140], _tol(dtype), "large sinks, the prompt")
    for p in range(140, 150):  # and decoded rows
        got = runner.step([StepEntry("a", [toks[p]], [0])]).cpu().numpy()
        assert_close(got[0], after[p], _tol(dtype), f"large sinks, decoded token {p}")


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("S", "float32"), ("Q", "bfloat16")])
def test_greedy_generation_through_the_engine(model_root, name, dtype):
    """`Engine.generate`: scheduler, portions under a token budget, decoding, sampler.  In float32 the tokens are the
    plain model's greedy tokens; in bfloat16 every generated token is the plain model's choice or within its rounding."""
    from machserve_b200 import Engine

    d = make_model_dir(model_root, name)
    vocab = CASES[name]["config"]["vocab"]
    prompts = [random_tokens(vocab, n, 40 + n) for n in (3, 29, 14, 1, 50)]
    eng = Engine(str(d), dtype, capacity=4, prefill_rows=16, tpp=CASES[name]["page"], max_seq=128)
    outs = eng.generate(prompts, max_new_tokens=12)
    eng.runner.cache.check()
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        seq = list(prompt)
        for tok in out:
            logits = plain_logits(d, seq, bf16_weights=(dtype == "bfloat16"))[-1]
            best = int(np.argmax(logits))
            if dtype == "float32":
                assert tok == best, f"{name}: token {len(seq) - len(prompt)} of a prompt of {len(prompt)} is {tok}, the plain model's is {best}"
            else:
                assert logits[best] - logits[tok] <= 2 * BF16_TOL * max(1.0, np.abs(logits).max())
            seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_root, tmp_path, dtype):
    """bin/trace_run itself on a model folder of this design, as a user drives it."""
    import subprocess

    d = make_model_dir(model_root, "S")
    toks = random_tokens(CASES["S"]["config"]["vocab"], 60, 9)
    steps = trace_portions("a", toks, [20, 2, 17, 1, 1, 1, 18])
    cmd = [sys.executable, str(REPO / "bin" / "trace_run"), "--model", str(d), "--dtype", dtype, "--out", str(tmp_path),
           "--max-tokens", "64", "--page-size", "8"]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            assert proc.stdout.readline().strip() == f"done {st['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    vocab = CASES["S"]["config"]["vocab"]
    results = {st["step"]: np.fromfile(tmp_path / f"{st['step']}.f32", dtype="<f4").reshape(-1, vocab) for st in steps}
    assert_close(collect_rows(steps, results)["a"], _want(d, dtype, toks), _tol(dtype), f"trace_run {dtype}")
