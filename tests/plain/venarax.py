"""Plain, slow, whole-sequence numpy implementation of the Venarax decoder, one function per mechanism.

Written from the design's equations; it keeps no cache, computes a whole sequence at once in float64, and
imports nothing from the engine package: it is what the engine is compared with.

Notation: d the model width, T the tokens of the sequence, p the position of a token (from 0), W [out, in]
a matrix applied as x . W^T.
"""
from __future__ import annotations

import math

import numpy as np


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b, var the mean of squared deviations."""
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps), eps inside the root."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) for each position p."""
    p = np.asarray(positions, dtype=np.int64)
    return 1.0 + coef * np.log(((p + 1) // every + 1).astype(np.float64))


def rotate_pairs(x, positions, base, dims):
    """Interleaved rotary turn of the first `dims` coordinates of x [T, heads, n]: the pair (2i, 2i+1) is turned by
    the angle p * base^(-2i/dims); the coordinates from `dims` on pass unchanged."""
    x = np.array(x, dtype=np.float64)
    i = np.arange(dims // 2, dtype=np.float64)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2].copy(), x[..., 1:dims:2].copy()
    x[..., 0:dims:2] = u * c - v * s
    x[..., 1:dims:2] = v * c + u * s
    return x


def softmax_attend(scores, values, visible, sink=None):
    """scores [T, T] (query, key), values [T, n], visible [T, T] bool.  Softmax over the visible keys; with `sink`
    the denominator also holds exp(sink), which has no value."""
    out = np.zeros((scores.shape[0], values.shape[1]))
    for i in range(scores.shape[0]):
        js = np.nonzero(visible[i])[0]
        s = scores[i, js]
        m = s.max() if sink is None else max(s.max(), sink)
        e = np.exp(s - m)
        den = e.sum() + (0.0 if sink is None else math.exp(sink - m))
        out[i] = (e / den) @ values[js]
    return out


def causal_mask(t, window=None):
    i, j = np.arange(t)[:, None], np.arange(t)[None, :]
    return (j <= i) if window is None else ((j <= i) & (i - j < window))


def sink_attention(h, w, p, cfg, eps, positions=None):
    """The 'attention' mixer: grouped heads, unit-rms norm of the whole q and k projections with weights,
    query temperature by position, no rotation, causal, softmax with a sink per head."""
    t = h.shape[0]
    positions = np.arange(t) if positions is None else positions
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = unit_rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    k = unit_rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = h @ w[p + "v"].T
    q = q * query_temperature(positions, cfg["q_temp"]["coef"], cfg["q_temp"]["every"])[:, None]
    q, k, v = q.reshape(t, H, dk), k.reshape(t, G, dk), v.reshape(t, G, dv)
    vis = causal_mask(t)
    out = np.zeros((t, H, dv))
    for head in range(H):
        g = head // (H // G)
        out[:, head] = softmax_attend(q[:, head] @ k[:, g].T * cfg["scale"], v[:, g], vis, float(w[p + "sink"][head]))
    return out.reshape(t, H * dv) @ w[p + "o"].T


def latent_attention(h, w, p, cfg, eps, positions=None):
    """The 'latent_attention' mixer: keys and values are made from one latent per token; one rotated key part is
    shared by all heads; sliding window; sigmoid gate on the heads' outputs."""
    t = h.shape[0]
    positions = np.arange(t) if positions is None else positions
    H, dn, dr, dv, r = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    q = (h @ w[p + "q"].T).reshape(t, H, dn + dr)
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :r], eps) * w[p + "dkv.norm"]
    k_rot = rotate_pairs(down[:, None, r:], positions, cfg["rot"]["base"], cfg["rot"]["dims"])[:, 0]
    q_rot = rotate_pairs(q[..., dn:], positions, cfg["rot"]["base"], cfg["rot"]["dims"])
    k_plain = (c @ w[p + "uk"].T).reshape(t, H, dn)
    v = (c @ w[p + "uv"].T).reshape(t, H, dv)
    vis = causal_mask(t, cfg["mask"]["size"])
    out = np.zeros((t, H, dv))
    for head in range(H):
        s = (q[:, head, :dn] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * cfg["scale"]
        out[:, head] = softmax_attend(s, v[:, head], vis)
    gate = 1.0 / (1.0 + np.exp(-(h @ w[p + "g"].T)))
    return (out.reshape(t, H * dv) * gate) @ w[p + "o"].T


def clamped_gated_mlp(h, w, p, limit):
    """g = min(gate(h), limit), u = clamp(up(h), -limit, limit); down(g * sigmoid(1.702 g) * (u + 1))."""
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)) @ w[p + "down"].T


MIXERS = {"attention": sink_attention, "latent_attention": latent_attention}


def layer(x, w, i, spec, eps):
    """Parallel layer: x + (mixer(norm1(x)) + mlp(norm2(x))), both norms of the same x."""
    p = f"l{i}."
    a = MIXERS[spec["type"]](layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps), w, p + "mix.", spec["mixer"], eps)
    if spec.get("mlp") is None:
        return x + a
    assert spec["mlp"]["kind"] == "dense"
    f = clamped_gated_mlp(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.", spec["mlp"]["limit"])
    return x + (a + f)


def run_order(config):
    """[(layer, pass number or None)]: layers start..stop-1 run `times` times in a row, the others once."""
    n, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return ([(i, None) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)]
            + [(i, None) for i in range(b, n)])


def forward(config, w, tokens, taps=None):
    """Logits [T, vocab] of a whole sequence; `taps`, a list, receives the stream after every run of a layer."""
    w = {k: np.asarray(v, dtype=np.float64) if np.asarray(v).dtype.kind == "f" else np.asarray(v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens, dtype=np.int64)]
    x = x0.copy()
    loop = config.get("loop")
    for i, t in run_order(config):
        if t is not None and i == loop["start"]:  # entry of a pass: mix with the embedding output, add the pass's vector
            x = np.concatenate([x, x0], axis=-1) @ w["loop.in"].T + w["loop.step"][t]
        x = layer(x, w, i, config["layers"][i], eps)
        if taps is not None:
            taps.append(x.copy())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
