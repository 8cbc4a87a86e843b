"""What the mixers with wide or unequal key and value rows share: the work lists of their tensor-core attention kernel,
and the choice between it and the exact kernel."""
from __future__ import annotations

import torch

from .. import ops
from .base import WorkPlan

PLAN = "row_tiles"    # the key of the work lists: every such mixer of a model shares them
TILES = (128, 64, 32, 16)  # rows of a portion that one block attends: 128 in the tcgen05 kernel, else by the width of the values
CONTEXT_BUCKET = 512  # a decoding row's run of keys is chosen from the longest context rounded up to this
BLOCKS_PER_SM = 6     # decoding rows are cut into runs of keys until the launch has about this many blocks per SM


def plan_words(max_rows: int, max_seqs: int) -> int:
    return 4 * max_seqs + 16 + sum(2 * (max_rows // t + max_seqs + 8) for t in TILES)


def plan(step) -> WorkPlan:
    """Rows that are alone in their sequence (decoding) go to the form whose 16 rows are the query heads of a token;
    portions of prompts are cut into tiles of up to 64, 32 and 16 consecutive rows (a list for each size)."""
    single = []
    t0, tn = {t: [] for t in TILES}, {t: [] for t in TILES}
    longest = longest_portion = key_tiles = 0
    for row, n, start in zip(step.row0, step.count, step.start):
        if n == 0:
            continue
        if n == 1:
            single.append(row)
            longest = max(longest, start + 1)
        else:
            longest_portion = max(longest_portion, start + n)
            for a in range(0, n, 128):  # tiles of 128 keys that the tiles of 128 rows see, in all
                key_tiles += (start + a + min(128, n - a) - 1) // 128 + 1
            for t in TILES:
                for a in range(0, n, t):
                    t0[t].append(row + a)
                    tn[t].append(min(t, n - a))
    cls = -(-longest // CONTEXT_BUCKET)
    cls_portion = -(-longest_portion // CONTEXT_BUCKET)
    mean_tiles = -(-key_tiles // (2 * len(t0[128]))) * 2 if t0[128] else 0
    if step.bucketed:  # lists of a few lengths (an entry of no rows does nothing), the context class a power of two
        for t in TILES:
            pad = -len(t0[t]) % (512 // t)
            t0[t] += [0] * pad
            tn[t] += [0] * pad
        if single:
            want = 16
            while want < len(single):
                want *= 4
            single += [-1] * (want - len(single))
        cls = 1 << (cls - 1).bit_length() if cls > 0 else 0
        cls_portion = 1 << (cls_portion - 1).bit_length() if cls_portion > 0 else 0
        mean_tiles = 4 * cls_portion  # (the bound that the portions' class gives: 512 keys are 4 tiles)
    lists = {"single_rows": single}
    for t in TILES:
        lists[f"tile{t}_row0"], lists[f"tile{t}_rows"] = t0[t], tn[t]
    return WorkPlan(lists, (cls, cls_portion, mean_tiles))


def supports(rt, dk: int, dv: int, vw: int, separate_v: bool) -> bool:
    return rt.dtype == torch.bfloat16 and ops.attention_wide_mma_supports(dk, dv, vw, separate_v)


def tcgen05_covers(rt, dk: int, dv: int, page_size: int) -> bool:
    """Whether portions of prompts can go to the framework's tcgen05 attention: keys and values of one width, 64 or 128."""
    return rt.dtype == torch.bfloat16 and dk == dv and dk in (64, 128) and ops.attention_prefill_tc_supports(dk, page_size)


def attend_portions_tcgen05(ctx, rt, table, q_half, k_pages, v_pages, out, sinks, hq: int, hkv: int, hd: int, window, scale: float):
    """The rows of prompt portions on the tcgen05 kernel, in tiles of 128 rows; the kernel's own plan says into how many
    runs the key tiles of a tile of rows are cut so that the launch fills the GPU."""
    work = ctx.work[PLAN]
    n_tiles = work.sizes["tile128_row0"]
    if not n_tiles:
        return out
    max_keys = work.shape[1] * CONTEXT_BUCKET
    if window:
        max_keys = min(max_keys, window + 128)
    splits, alone, run_tiles = ops.attention_prefill_tc_plan(n_tiles, hq, hkv, hd, max_keys, work.shape[2] * n_tiles)
    scratch = counters = None
    if splits > 1:
        words = ops.attention_prefill_tc_scratch_words(n_tiles, hq, hd, splits)
        scratch = rt.workspace.get("wide_attend.tc_splits", (words,), torch.float32)
        counters = rt.workspace.get("wide_attend.tc_counters", (n_tiles * hq,), torch.int32, zero=True)
    return ops.attention_prefill_tc(q_half, k_pages, v_pages, out, work.lists["tile128_row0"], work.lists["tile128_rows"], n_tiles,
                                    ctx.positions, ctx.slot_of_token, table, hq, hkv, hd, window, scale, splits, scratch, counters,
                                    alone=alone, run_tiles=run_tiles, sinks=sinks)


def cluster_covers(rt, dk: int, dv: int, groups: int) -> bool:
    """Whether decoding rows can go to the framework's cluster kernel: keys and values of one width that it is built for."""
    return rt.dtype == torch.bfloat16 and dk == dv and ops.attention_decode_supports(dk, groups) and ops.attention_prefill_supports(dk)


def attend_single_cluster(ctx, rt, launch_cache: dict, table, q_half, k_pages, v_pages, out, sinks, hq: int, hkv: int, hd: int, window,
                          scale: float):
    """Rows that are alone in their sequences on the framework's decode kernel (a cluster of blocks per row and key head,
    the launch by the rules measured for it), with the sink in its merge."""
    from .attention import decode_launch

    work = ctx.work[PLAN]
    t = work.sizes["single_rows"]
    tiles = (work.shape[0] * CONTEXT_BUCKET + 63) // 64
    if window:
        tiles = min(tiles, (window + 63) // 64 + 1)
    splits, stages, warps, kpw, parts = decode_launch(rt, hd, ops.attention_decode_cluster_max_stages(hd), launch_cache, t * hkv, tiles)
    scratch = counters = None
    if parts > 1:
        words = ops.attention_decode_cluster_scratch_words(t, hq, hkv, hd, parts)
        scratch = rt.workspace.get("wide_attend.decode_parts", (words,), torch.float32)
        counters = rt.workspace.get("wide_attend.decode_counters", (t * hkv,), torch.int32, zero=True)
    every_row = work.sizes["tile128_row0"] == 0 and t == q_half.shape[0]
    return ops.attention_decode_cluster(q_half, k_pages, v_pages, out, ctx.positions, ctx.slot_of_token, table, hq, hkv, hd, window, scale,
                                        splits, stages, rows=None if every_row else work.lists["single_rows"], num_rows=t, warps=warps,
                                        keys_per_warp=kpw, parts=parts, scratch=scratch, counters=counters, sinks=sinks)


def attend(ctx, rt, fast: bool, table, q, k_pages, v_pages, out, sinks, hq: int, hkv: int, dk: int, dv: int, window, scale: float,
           q_half=None, tcgen05: bool = False, cluster=None, score=None):
    """Every row of q over its sequence's pages: on the tensor cores when the widths allow it in bfloat16 (decoding rows
    with their key tiles cut into as many runs as fill the GPU, portions in tiles of 64, 32 or 16 rows), else the exact kernel.
    With `q_half` (the queries in bfloat16) the framework's own kernels for keys and values of one width take what they
    cover: `cluster` (a dict for the launch rules' results) sends decoding rows to its cluster kernel, `tcgen05` the
    portions to its tcgen05 kernel; both add the sinks themselves.  `score` (`ops.ScoreExtras`: a soft cap, a bias by head
    and distance, a mask by chunks) is applied by the exact and the mma.sync kernels; the other two do not have it."""
    if score is not None and (tcgen05 or cluster is not None):
        raise ValueError("the tcgen05 and cluster attention kernels have no soft cap, distance bias or chunks")
    if not fast:
        return ops.attention_wide(q, k_pages, v_pages, out, sinks, ctx.positions, ctx.slot_of_token, table, hq, hkv,
                                  dk, dv, window, scale, share_rows=ctx.max_query_len > 1, score=score)
    work = ctx.work[PLAN]
    tile = ops.attention_wide_mma_tile_rows(dv)
    singles, tiles = work.sizes["single_rows"], work.sizes[f"tile{tile}_row0"]
    if singles and cluster is not None and q_half is not None:
        attend_single_cluster(ctx, rt, cluster, table, q_half, k_pages, v_pages, out, sinks, hq, hkv, dk, window, scale)
    elif singles:
        items = singles * hkv * (-(-(hq // hkv) // 16))
        keys = work.shape[0] * CONTEXT_BUCKET
        if window:
            keys = min(keys, window + 63)
        if score is not None and score.chunk:
            keys = min(keys, score.chunk + 63)
        splits = max(1, min(BLOCKS_PER_SM * rt.sm_count // items, -(-keys // 64), 32))
        scratch = None
        if splits > 1:
            scratch = rt.workspace.get("wide_attend.splits", (ops.attention_wide_mma_scratch_words(items, dv, splits),), torch.float32)
        rows = None if tiles == 0 and singles == q.shape[0] else work.lists["single_rows"]
        ops.attention_wide_mma(q, k_pages, v_pages, out, sinks, ctx.positions, ctx.slot_of_token, table, rows, None, singles, True,
                               hq, hkv, dk, dv, window, scale, splits, scratch, score=score)
    if tcgen05 and q_half is not None:  # portions on the tcgen05 kernel (the part has made sure that it covers the sizes)
        attend_portions_tcgen05(ctx, rt, table, q_half, k_pages, v_pages, out, sinks, hq, hkv, dk, window, scale)
    elif tiles:
        ops.attention_wide_mma(q, k_pages, v_pages, out, sinks, ctx.positions, ctx.slot_of_token, table, work.lists[f"tile{tile}_row0"],
                               work.lists[f"tile{tile}_rows"], tiles, False, hq, hkv, dk, dv, window, scale, score=score)
    return out


class WideAttendPlan:
    """Mixin of the mixers that attend through `attend`: their shared work lists."""

    def plan_key(self):
        return PLAN

    def plan(self, step):
        return plan(step)

    def plan_words(self, max_rows, max_seqs):
        return plan_words(max_rows, max_seqs)
