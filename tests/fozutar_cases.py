"""Tiny Fozutar configurations for the tests, and how their model folders are made.

They differ from one another in every size and constant: one, two, three and four query heads per key head, chunks that are
and are not multiples of the page size and of the kernels' key tiles, bias tables of several sizes and reaches, soft caps
from tight to loose, decay ranks and time constants, dense and routed feed-forwards (one expert of several, all of them, a
few), a layer without a feed-forward, loops that start after the first layer, cover everything, run once, and no loop.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np


def _attention(heads, kv_heads, dim, scale, softcap, bias_rows, bias_max, chunk):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
                                           "softcap": softcap, "bias_rows": bias_rows, "bias_max": bias_max, "mask": {"size": chunk}}}


def _gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _config(vocab, width, eps, scale, positions, layers, loop=None):
    out = {"architecture": "Fozutar", "vocab": vocab, "width": width, "max_positions": positions, "norm": {"eps": eps},
           "embedding": {"scale": scale}, "layers": layers}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CASES = {
    # a loop that starts after the first layer; chunks of 20 and 7 tokens (no multiples of a page); a layer without a feed-forward
    "A": dict(config=_config(150, 64, 1e-5, 3.0, 256, [
        {**_gla(2, 16, 24, 8.0, 4), "mlp": _moe(32, 5, 2)},
        {**_attention(4, 2, 16, 0.3, 5.0, 8, 40, 20), "mlp": _dense(96)},
        {**_attention(3, 3, 8, 0.5, 30.0, 6, 12, 7), "mlp": None},
        {**_gla(3, 8, 12, 2.0, 3), "mlp": _dense(48)},
    ], (1, 3, 2)), seed=21, page=8),
    # no loop; one key head for all query heads; a single head; an odd key size; a chunk of one page, and one longer than the prompts
    "B": dict(config=_config(200, 48, 1e-6, 1.0, 300, [
        {**_attention(6, 1, 7, 0.4, 2.0, 10, 100, 16), "mlp": _moe(24, 3, 3)},
        {**_gla(1, 10, 10, 32.0, 2), "mlp": _moe(40, 7, 1)},
        {**_attention(1, 1, 32, 0.2, 100.0, 4, 9, 500), "mlp": _dense(64)},
        {**_gla(4, 8, 16, 1.0, 8), "mlp": None},
    ]), seed=22, page=16),
    # a loop over all layers that runs once; widths that the bfloat16 engine's tensor-core attention covers; a chunk of 64
    "C": dict(config=_config(128, 96, 1e-6, 8.0, 512, [
        {**_attention(4, 1, 32, 0.17, 20.0, 16, 64, 64), "mlp": _moe(64, 8, 2)},
        {**_gla(2, 32, 40, 16.0, 8), "mlp": _dense(128)},
    ], (0, 2, 1)), seed=23, page=16),
    # three passes over a looped pair; as many query heads as key heads; chunk 33 (one past a key tile)
    "D": dict(config=_config(144, 64, 1e-5, 5.0, 256, [
        {**_gla(2, 12, 20, 4.0, 5), "mlp": _moe(48, 4, 2)},
        {**_attention(2, 2, 16, 0.25, 10.0, 12, 30, 33), "mlp": _moe(32, 6, 4)},
        {**_attention(8, 2, 48, 0.14, 50.0, 20, 90, 48), "mlp": _dense(80)},
    ], (0, 2, 3)), seed=24, page=8),
    # odd sizes everywhere: a width, feed-forwards, vocabulary and head sizes that no vector access and no tensor-core tile fits
    "E": dict(config=_config(131, 50, 1e-6, 2.5, 200, [
        {**_gla(3, 7, 9, 3.0, 3), "mlp": _moe(21, 5, 2)},
        {**_attention(5, 1, 5, 0.45, 7.0, 7, 25, 13), "mlp": _dense(37)},
    ], (1, 2, 2)), seed=25, page=8),
    # recurrent layers only (no pages at all), the whole model looped twice
    "F": dict(config=_config(120, 32, 1e-5, 4.0, 256, [
        {**_gla(2, 8, 16, 12.0, 4), "mlp": _dense(64)},
        {**_gla(1, 16, 8, 6.0, 2), "mlp": _moe(32, 4, 2)},
    ], (0, 2, 2)), seed=26, page=8),
    # attention layers only (no state at all), no loop
    "G": dict(config=_config(90, 48, 1e-6, 1.5, 256, [
        {**_attention(3, 1, 16, 0.25, 8.0, 10, 60, 24), "mlp": _moe(32, 4, 1)},
        {**_attention(2, 2, 8, 0.4, 40.0, 4, 20, 10), "mlp": _dense(96)},
    ]), seed=27, page=16),
}


def make_model_dir(root, name: str, steady_routers: bool = False) -> Path:
    """Writes the tiny model `name` (config.json, model.safetensors in bfloat16-exact float32) under root.
    `steady_routers`: a second folder whose routers weigh the token 30 times less against their biases: most tokens then go
    the way the biases say, by margins that rounding to bfloat16 cannot turn, and some still go their own way.  (The
    float32 tests use the routers as they are drawn, where every token goes its own way.)"""
    import torch

    from machserve_b200.config import config_from_json
    from machserve_b200.weights import write_random_model
    from machserve_b200.weights.safetensors_io import write_safetensors

    case = CASES[name]
    out = Path(root) / f"fozutar_{name}"
    if not (out / "model.safetensors").exists():
        # large deviations: logits that separate, so that a dropped key or a wrong row shows
        write_random_model(config_from_json(case["config"]), out, case["seed"], torch.float32, 0.12, 0.3, 0.1)
    if not steady_routers:
        return out
    steady = Path(root) / f"fozutar_{name}_steady"
    if not (steady / "model.safetensors").exists():
        steady.mkdir(parents=True, exist_ok=True)
        _, w = read_weights(out)
        tensors = {}
        for k, v in w.items():
            t = torch.from_numpy(np.asarray(v, dtype=np.float32) if np.asarray(v).dtype.kind == "f" else np.asarray(v))
            if k.endswith("mlp.router"):
                t = (t / 30.0).to(torch.bfloat16).to(torch.float32)
            tensors[k] = t
        (steady / "config.json").write_text((out / "config.json").read_text())
        write_safetensors(steady / "model.safetensors", tensors)
    return steady


def read_weights(model_dir, round_to_bf16: bool = False):
    from tests.plain import read_model_dir

    return read_model_dir(model_dir, round_to_bf16=round_to_bf16)


def plain_logits(model_dir, tokens, bf16_weights: bool = False) -> np.ndarray:
    from tests.plain.fozutar import forward

    cfg, w = read_weights(model_dir, bf16_weights)
    return forward(cfg, w, tokens)


CLOSE_CALL = 0.01  # a router margin below this can fall either way under bfloat16 rounding (steady routers)


def plain_logits_and_close_calls(model_dir, tokens, bf16_weights: bool = False, tol: float = 0.02):
    """(logits [T, vocab], unsure [T] bool).  `unsure[t]` says that the plain model itself cannot vouch for row t under
    bfloat16 rounding: some router chose between two experts by less than CLOSE_CALL at token t (an engine that rounds
    may rightly choose the other), or the row's logits move by more than `tol` (times their largest) when nothing but
    the layers' normed inputs are rounded to bfloat16 (a recurrent head whose few live terms cancel, for instance, is
    then divided by a root mean square that is all rounding)."""
    import torch

    from tests.plain.fozutar import forward

    cfg, w = read_weights(model_dir, bf16_weights)
    margins = []
    logits = forward(cfg, w, tokens, None, margins)
    unsure = np.zeros(len(tokens), dtype=bool)
    for m in margins:
        unsure |= m < CLOSE_CALL
    rounded = forward(cfg, w, tokens, None, None, lambda h: torch.from_numpy(h.astype(np.float32)).to(torch.bfloat16).to(torch.float64).numpy())
    unsure |= np.abs(rounded - logits).max(-1) > tol * max(1.0, float(np.abs(logits).max()))
    return logits, unsure
