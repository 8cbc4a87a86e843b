"""Plain, slow, whole-sequence numpy implementation of the Fozutar decoder, one function per mechanism.

Written from the design's equations; it keeps no cache and no state between calls, computes a whole sequence at once
in float64, and imports nothing from the engine package: it is what the engine is compared with.

Notation: d the model width, T the tokens of the sequence, p the position of a token (from 0), W [out, in] a matrix
applied as x . W^T.
"""
from __future__ import annotations

import math

import numpy as np


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, eps inside the root."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def embed(tokens, table, scale, pos_table):
    """Scaled token rows plus the (unscaled) learned vector of each position."""
    t = np.asarray(tokens, dtype=np.int64)
    return table[t] * scale + pos_table[np.arange(len(t))]


def distance_row(n, rows, reach):
    """Which row of a bias table of `rows` rows distance n reads: n itself below rows // 2, then logarithmic steps up to
    `reach`, the last row beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))


def chunk_mask(t, size):
    """visible[i, j]: j <= i and both in the same chunk of `size` positions counted from position 0."""
    i, j = np.arange(t)[:, None], np.arange(t)[None, :]
    vis = j <= i
    return vis if size is None else vis & (i // size == j // size)


def soft_cap(s, cap):
    return cap * np.tanh(s / cap)


def chunked_attention(h, w, p, cfg, eps):
    """Grouped heads; q and k with biases; v is k as projected; q and k normed per head without a weight; capped scores
    plus a bias by distance and head; chunked causal mask; softmax; output projection."""
    t = h.shape[0]
    H, G, dk = cfg["heads"], cfg["kv_heads"], cfg["dim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(t, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(t, G, dk)
    v = k
    qn, kn = unit_rms(q, eps), unit_rms(k, eps)
    rel = w[p + "rel"]
    rows = rel.shape[0]
    dist = np.arange(t)[:, None] - np.arange(t)[None, :]
    row_of = np.array([distance_row(n, rows, cfg["bias_max"]) for n in range(t)])
    which = row_of[np.clip(dist, 0, None)]
    vis = chunk_mask(t, cfg.get("mask", {}).get("size") if cfg.get("mask") else None)
    out = np.zeros((t, H, dk))
    for head in range(H):
        g = head // (H // G)
        s = soft_cap(qn[:, head] @ kn[:, g].T * cfg["scale"], cfg["softcap"]) + rel[which, head]
        s = np.where(vis, s, -np.inf)
        e = np.exp(s - s.max(-1, keepdims=True))
        out[:, head] = (e / e.sum(-1, keepdims=True)) @ v[:, g]
    return out.reshape(t, H * dk) @ w[p + "o"].T


def log_decay(h, w, p, tau):
    """ln of sigmoid(z)^(1/tau), z the low-rank projection with its bias."""
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    return -np.logaddexp(0.0, -z) / tau


def gla_recurrence(q, k, v, g, state=None):
    """q, k, g [T, dk]; v [T, dv].  S <- exp(g_t)[:, None] * S + outer(k_t, v_t); o_t = S^T q_t.  Returns (o, S)."""
    dk, dv = q.shape[1], v.shape[1]
    s = np.zeros((dk, dv)) if state is None else state.copy()
    o = np.zeros((q.shape[0], dv))
    for t in range(q.shape[0]):
        s = np.exp(g[t])[:, None] * s + np.outer(k[t], v[t])
        o[t] = s.T @ q[t]
    return o, s


def gated_linear_attention(h, w, p, cfg, eps):
    t = h.shape[0]
    H, dk, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    q = (h @ w[p + "q"].T).reshape(t, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(t, H, dk)
    v = (h @ w[p + "v"].T).reshape(t, H, dv)
    g = log_decay(h, w, p, cfg["tau"]).reshape(t, H, dk)
    o = np.zeros((t, H, dv))
    for head in range(H):
        o[:, head], _ = gla_recurrence(q[:, head], k[:, head], v[:, head], g[:, head])
    o = rms_norm(o, w[p + "norm"], eps)
    return (o.reshape(t, H * dv) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def dense_mlp(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, top, margins=None):
    """(ids [T, top], weights [T, top]): the experts with the largest router logits, softmax over the chosen logits.
    `margins`, a list, receives [T]: by how much the last chosen logit is ahead of the best one that was not chosen."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    order = np.argsort(-z, axis=-1, kind="stable")
    ids = order[:, :top]
    chosen = np.take_along_axis(z, ids, -1)
    if margins is not None:
        nxt = np.take_along_axis(z, order[:, top : top + 1], -1)[:, 0] if top < z.shape[1] else np.full(z.shape[0], -np.inf)
        margins.append(chosen[:, -1] - nxt)
    e = np.exp(chosen - chosen.max(-1, keepdims=True))
    return ids, e / e.sum(-1, keepdims=True)


def routed_mlp(h, w, p, cfg, margins=None):
    ids, weights = route(h, w, p, cfg["router"]["top"], margins)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], weights[t]):
            q = f"{p}e{int(e)}."
            out[t] += a * ((silu(w[q + "gate"] @ h[t]) * (w[q + "up"] @ h[t])) @ w[q + "down"].T)
    return out


def feed_forward(h, w, p, cfg, margins=None):
    if cfg is None:
        return 0.0
    return dense_mlp(h, w, p) if cfg["kind"] == "dense" else routed_mlp(h, w, p, cfg, margins)


MIXERS = {"attention": chunked_attention, "gla": gated_linear_attention}


def layer(x, w, i, spec, eps, margins=None, round_h=None):
    """One norm, read by both halves: x + (mixer(h) + ff(h)), h = norm1(x).  `round_h`, a function, is applied to h: what
    an engine does that hands the normed rows on in fewer bits."""
    p = f"l{i}."
    h = rms_norm(x, w[p + "norm1"], eps)
    if round_h is not None:
        h = round_h(h)
    return x + (MIXERS[spec["type"]](h, w, p + "mix.", spec["mixer"], eps) + feed_forward(h, w, p + "mlp.", spec.get("mlp"), margins))


def run_order(config):
    """[(layer, pass number or None)]: layers start..stop-1 run `times` times in a row, the others once."""
    n, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return ([(i, None) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)]
            + [(i, None) for i in range(b, n)])


def forward(config, w, tokens, taps=None, margins=None, round_h=None):
    """Logits [T, vocab] of a whole sequence; `taps`, a list, receives the stream after every run of a layer; `margins`, a
    list, receives for every run of a routed feed-forward the router's margins [T] (see `route`)."""
    w = {k: np.asarray(v, dtype=np.float64) if np.asarray(v).dtype.kind == "f" else np.asarray(v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x0 = embed(tokens, w["embed"], config.get("embedding", {}).get("scale", 1.0), w["pos"])
    x = x0.copy()
    loop = config.get("loop")
    for i, t in run_order(config):
        if t is not None and i == loop["start"]:  # the start of a pass
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        x = layer(x, w, i, config["layers"][i], eps, margins, round_h)
        if taps is not None:
            taps.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T
