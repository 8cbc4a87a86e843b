"""Tiny Venarax configurations for the tests, and how their model folders are made.

The configurations differ from one another in every size and constant: key and value sizes per head that differ,
one, two and three query heads per key head, a rotation over all and over part of the rotated coordinates, windows
that are and are not multiples of the page size, a temperature period of a few tokens (so that it changes inside
every test), two clamp limits, a layer without a feed-forward, a loop that starts after the first layer, a loop
over all layers that runs once, and no loop.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np


def _attention(heads, kv_heads, dim, vdim, scale, coef, every):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "q_temp": {"coef": coef, "every": every}}}


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, dims, window):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "scale": scale, "rot": {"base": base, "dims": dims}, "mask": {"size": window}}}


def _mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


CASES = {
    # a loop that starts after the first layer; key and value sizes differ everywhere; partial rotation in layer 3
    "P": dict(
        config={
            "architecture": "Venarax", "vocab": 160, "width": 64, "norm": {"eps": 1e-5},
            "layers": [
                {**_latent(2, 16, 8, 24, 32, 0.2, 1000.0, 8, 11), "mlp": _mlp(96, 1.5)},
                {**_attention(4, 2, 24, 16, 0.15, 0.7, 8), "mlp": _mlp(80, 0.7)},
                {**_attention(3, 3, 8, 12, 0.3, 0.4, 5), "mlp": None},
                {**_latent(3, 12, 6, 8, 20, 0.25, 50.0, 4, 7), "mlp": _mlp(72, 1.5)},
            ],
            "loop": {"start": 1, "stop": 3, "times": 2},
        },
        seed=11, page=8,
    ),
    # no loop; one key head for all query heads; a single head; an odd key size; a window of one page and of one token
    "Q": dict(
        config={
            "architecture": "Venarax", "vocab": 200, "width": 48, "norm": {"eps": 1e-6},
            "layers": [
                {**_attention(6, 1, 7, 20, 0.35, 0.5, 3), "mlp": _mlp(64, 2.5)},
                {**_latent(1, 10, 4, 10, 16, 0.3, 10000.0, 4, 16), "mlp": _mlp(40, 1.0)},
                {**_latent(4, 8, 8, 16, 24, 0.2, 300.0, 2, 1), "mlp": _mlp(56, 2.5)},
                {**_attention(1, 1, 32, 16, 0.18, 1.1, 16), "mlp": _mlp(64, 2.5)},
            ],
        },
        seed=12, page=16,
    ),
    # a loop over all layers that runs once, and wider values than the small kernels' 64 and 128
    "R": dict(
        config={
            "architecture": "Venarax", "vocab": 128, "width": 96, "norm": {"eps": 1e-6},
            "layers": [
                {**_attention(2, 1, 16, 144, 0.2, 0.3, 7), "mlp": _mlp(128, 2.0)},
                {**_latent(2, 24, 16, 40, 136, 0.12, 20000.0, 16, 40), "mlp": _mlp(128, 2.0)},
            ],
            "loop": {"start": 0, "stop": 2, "times": 1},
        },
        seed=13, page=16,
    ),
    # three passes over a looped pair, as many query heads as key heads
    "S": dict(
        config={
            "architecture": "Venarax", "vocab": 144, "width": 64, "norm": {"eps": 1e-5},
            "layers": [
                {**_attention(2, 2, 16, 16, 0.25, 0.6, 4), "mlp": _mlp(64, 1.2)},
                {**_latent(2, 8, 8, 12, 24, 0.3, 100.0, 8, 20), "mlp": _mlp(64, 1.2)},
                {**_attention(4, 1, 12, 20, 0.2, 0.2, 9), "mlp": _mlp(48, 3.0)},
            ],
            "loop": {"start": 0, "stop": 2, "times": 3},
        },
        seed=14, page=8,
    ),
    # widths that the bfloat16 engine's tensor-core attention covers in every layer (key rows in steps of 16, value rows
    # in steps of 8), a window that is no multiple of a tile of keys, more query heads per key head than a tile has rows
    "T": dict(
        config={
            "architecture": "Venarax", "vocab": 176, "width": 64, "norm": {"eps": 1e-6},
            "layers": [
                {**_attention(4, 2, 32, 16, 0.18, 0.5, 6), "mlp": _mlp(96, 2.0)},
                {**_latent(3, 16, 16, 24, 48, 0.2, 5000.0, 16, 37), "mlp": _mlp(64, 2.0)},
                {**_attention(18, 1, 16, 8, 0.25, 0.3, 11), "mlp": _mlp(64, 1.0)},
            ],
            "loop": {"start": 1, "stop": 2, "times": 2},
        },
        seed=15, page=16,
    ),
    # key and value rows of 64 in an attention layer: the sizes at which the bfloat16 engine sends the portions of prompts
    # to its tcgen05 attention (with the sink) and decoding rows to the mma.sync kernel
    "U": dict(
        config={
            "architecture": "Venarax", "vocab": 192, "width": 128, "norm": {"eps": 1e-6},
            "layers": [
                {**_attention(4, 2, 64, 64, 0.125, 0.4, 10), "mlp": _mlp(160, 2.0)},
                {**_latent(2, 32, 16, 32, 48, 0.15, 10000.0, 16, 70), "mlp": _mlp(96, 2.0)},
            ],
            "loop": {"start": 0, "stop": 1, "times": 2},
        },
        seed=16, page=16,
    ),
    # odd sizes everywhere: a width, feed-forward, vocabulary and head sizes that no vector access and no tensor-core tile fits
    "V": dict(
        config={
            "architecture": "Venarax", "vocab": 131, "width": 50, "norm": {"eps": 1e-6},
            "layers": [
                {**_latent(3, 7, 6, 9, 10, 0.3, 777.0, 6, 13), "mlp": _mlp(37, 1.7)},
                {**_attention(5, 1, 5, 3, 0.4, 0.9, 7), "mlp": _mlp(41, 1.7)},
            ],
            "loop": {"start": 1, "stop": 2, "times": 2},
        },
        seed=17, page=8,
    ),
}


def make_model_dir(root, name: str) -> Path:
    """Writes the tiny model `name` (config.json, model.safetensors in bfloat16-exact float32) under root."""
    import torch

    from machserve_b200.config import config_from_json
    from machserve_b200.weights import write_random_model

    case = CASES[name]
    out = Path(root) / f"venarax_{name}"
    if not (out / "model.safetensors").exists():
        # large deviations: logits that separate, so that a dropped key or a wrong row shows
        write_random_model(config_from_json(case["config"]), out, case["seed"], torch.float32, 0.12, 0.3, 0.1)
    return out


def read_weights(model_dir, round_to_bf16: bool = False):
    from tests.plain import read_model_dir

    return read_model_dir(model_dir, round_to_bf16=round_to_bf16)


def plain_logits(model_dir, tokens, bf16_weights: bool = False) -> np.ndarray:
    from tests.plain.venarax import forward

    cfg, w = read_weights(model_dir, bf16_weights)
    return forward(cfg, w, tokens)
