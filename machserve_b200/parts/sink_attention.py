"""Grouped-query attention without rotation: query/key norm over the whole projection, a query temperature that
grows with the position, and a learned sink in every head's softmax."""
from __future__ import annotations

import torch

from .. import ops
from . import wide_attend
from ..weights.loader import TensorDecl
from .base import CachePlane, Mixer, PagedCache, matrix, register_mixer, vector_f32


@register_mixer("sink_attention")
class SinkAttention(wide_attend.WideAttendPlan, Mixer):
    """q = Wq x, k = Wk x, v = Wv x (no biases, one product).  The whole q row and the whole k row are each divided by
    their root mean square (eps inside the root) and multiplied by a weight of their own, before they are split into
    heads.  The query at position p is then multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).  Positions enter
    nowhere else.  Query head h reads key/value head h // (heads / kv_heads); score = scale * q . k over the keys
    0..p (or the last `window`); the softmax's denominator also holds exp(sink_h), a learned number per head that has no
    value and is not scaled.  Keys have `key_dim` and values `value_dim` coordinates per head; the output projection
    reads the heads' values side by side.  Norms, temperature, scores and softmax are float32; the query stays float32
    up to the scores (the exact kernel) or is rounded to bfloat16 as it enters the tensor core (bfloat16 runtime, widths
    the tensor-core kernel covers); the delta is float32.

    params: prefix, hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, eps, temp_coef (0: none),
    temp_every, window (or None), sink (False: a plain softmax).  Tensors under the prefix: q, k, v, o (matrices),
    q.norm, k.norm (weights over the whole projections), sink [heads].
    """

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden = int(spec["hidden_size"])
        self.hq, self.hkv = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.dk, self.dv = int(spec["key_dim"]), int(spec["value_dim"])
        if self.hq % self.hkv:
            raise ValueError(f"sink_attention: {self.hq} heads are not a multiple of {self.hkv} kv heads")
        if self.dv > 512:
            raise ValueError(f"sink_attention: values of {self.dv} coordinates per head are more than the kernel covers (512)")
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.coef, self.every = float(spec.get("temp_coef", 0.0)), int(spec.get("temp_every", 1))
        self.window = spec.get("window")
        self.has_sink = bool(spec.get("sink", True))
        self.qw, self.kw, self.vw = self.hq * self.dk, self.hkv * self.dk, self.hkv * self.dv

    def cache_need(self):
        return PagedCache((CachePlane("k", self.hkv, self.dk), CachePlane("v", self.hkv, self.dv)), self.window)

    def tensors(self):
        p = self.prefix
        out = [
            TensorDecl(p + "q", (self.qw, self.hidden)), TensorDecl(p + "k", (self.kw, self.hidden)),
            TensorDecl(p + "v", (self.vw, self.hidden)), TensorDecl(p + "q.norm", (self.qw,), init="scale"),
            TensorDecl(p + "k.norm", (self.kw,), init="scale"), TensorDecl(p + "o", (self.hidden, self.hq * self.dv)),
        ]
        if self.has_sink:
            out.append(TensorDecl(p + "sink", (self.hq,), init="bias"))
        return out

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        self.w_qkv = matrix(torch.cat([tensors[p + "q"], tensors[p + "k"], tensors[p + "v"]], dim=0), rt)
        self.w_o = matrix(tensors[p + "o"], rt)
        self.q_norm, self.k_norm = vector_f32(tensors[p + "q.norm"]), vector_f32(tensors[p + "k.norm"])
        self.sinks = vector_f32(tensors[p + "sink"]) if self.has_sink else None
        self.fast = wide_attend.supports(rt, self.dk, self.dv, self.dv, True)  # bfloat16: the tensor-core kernel
        # keys and values of one width that the framework's decode kernel is built for: decoding rows go there
        self.cluster = {} if self.fast and wide_attend.cluster_covers(rt, self.dk, self.dv, self.hq // self.hkv) else None

    def forward(self, ctx, x, cache, owns_cache=True):
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        width = self.qw + (self.kw + self.vw if owns_cache else 0)
        proj = ws.get("sink_attn.qkv", (t, width), torch.float32)
        ops.linear(x, self.w_qkv[:width], None, proj)
        q = ws.get("sink_attn.q", (t, self.qw), torch.float32)
        k_pages, v_pages = cache.planes["k"], cache.planes["v"]
        table = cache.block_table(ctx)
        # the framework's kernels for keys and values of one width read bfloat16 queries: portions of prompts go to the tcgen05
        # kernel where it covers the sizes, decoding rows to the cluster kernel
        tcgen05 = self.fast and ctx.max_query_len > 1 and wide_attend.tcgen05_covers(rt, self.dk, self.dv, k_pages.shape[2])
        q_half = ws.get("sink_attn.q_half", (t, self.qw), rt.dtype) if tcgen05 or self.cluster is not None else None
        ops.qk_norm_store(proj, self.q_norm, self.k_norm, self.eps, self.coef, self.every, ctx.positions, ctx.slot_of_token, table,
                          q, k_pages, v_pages, self.hkv, self.dk, self.dv, store=owns_cache, q_half=q_half)
        out = ws.get("sink_attn.out", (t, self.hq * self.dv), rt.dtype)
        wide_attend.attend(ctx, rt, self.fast, table, q, k_pages, v_pages, out, self.sinks, self.hq, self.hkv, self.dk, self.dv,
                           self.window, self.scale, q_half=q_half, tcgen05=tcgen05, cluster=self.cluster)
        delta = ws.get("mixer.delta_f32", (t, self.hidden), torch.float32)
        return ops.linear(out, self.w_o, None, delta)
