"""Gated linear attention: a recurrent mixer with a matrix state per head and a learned decay per key channel."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import FixedState, Mixer, matrix, register_mixer, vector_f32


@register_mixer("gated_linear_attention")
class GatedLinearAttention(Mixer):
    """q = Wq x * key_dim^(-1/2), k = Wk x (heads x key_dim), v = Wv x (heads x value_dim); a decay per key channel
    a = sigmoid(z)^(1/tau), z = Wa2 (Wa1 x) + ba2 (a low-rank projection, heads x key_dim).  Per head and sequence

        S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,

    with S [key_dim, value_dim] zero at the start of a sequence, float32, carried from step to step in the request's state
    slot.  Each head's o_t is divided by its root mean square over value_dim (eps inside the root) and multiplied by a weight
    [value_dim] that the heads share; the heads side by side are multiplied by silu(Wg x) and go through Wo.  The five input
    projections are one product with a float32 result; the decay (through its logarithm), the state, the norm and the
    gate are float32.

    params: prefix, hidden_size, num_heads, key_dim, value_dim, decay_rank, tau, eps.  Tensors under the prefix: q, k, v, g,
    a1 [decay_rank, hidden], a2 [heads*key_dim, decay_rank], a2.b, norm [value_dim], o.
    """

    graph_safe = True
    kernel_files = ('gla',)

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden, self.heads = int(spec["hidden_size"]), int(spec["num_heads"])
        self.dk, self.dv, self.rank = int(spec["key_dim"]), int(spec["value_dim"]), int(spec["decay_rank"])
        self.tau, self.eps = float(spec["tau"]), float(spec["eps"])
        if self.dk > 256:
            raise ValueError(f"gated_linear_attention: {self.dk} key channels a head are more than the kernel covers (256)")
        self.kw, self.vw = self.heads * self.dk, self.heads * self.dv
        # columns of the one input product: q | k | v | g | a1
        self.q_off, self.k_off, self.v_off, self.g_off = 0, self.kw, 2 * self.kw, 2 * self.kw + self.vw
        self.a_off = self.g_off + self.vw
        self.width = self.a_off + self.rank

    def cache_need(self):
        return FixedState((self.heads, self.dk, self.dv))

    def tensors(self):
        p, h = self.prefix, self.hidden
        return [
            TensorDecl(p + "q", (self.kw, h)), TensorDecl(p + "k", (self.kw, h)), TensorDecl(p + "v", (self.vw, h)),
            TensorDecl(p + "g", (self.vw, h)), TensorDecl(p + "a1", (self.rank, h)), TensorDecl(p + "a2", (self.kw, self.rank)),
            TensorDecl(p + "a2.b", (self.kw,), init="bias"), TensorDecl(p + "norm", (self.dv,), init="scale"),
            TensorDecl(p + "o", (h, self.vw)),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        self.w_in = matrix(torch.cat([tensors[p + n] for n in ("q", "k", "v", "g", "a1")], dim=0), rt)
        self.w_a2 = matrix(tensors[p + "a2"], rt)
        self.b_a2 = vector_f32(tensors[p + "a2.b"])
        self.norm = vector_f32(tensors[p + "norm"])
        self.w_o = matrix(tensors[p + "o"], rt)

    def forward(self, ctx, x, cache, owns_cache=True):
        if not owns_cache:
            raise ValueError("gated_linear_attention: a run cannot read another run's state")
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        proj = ws.get("gla.proj", (t, self.width), torch.float32)
        ops.linear(x, self.w_in, None, proj)
        decay = ws.get("gla.decay", (t, self.kw), torch.float32)
        ops.gla_decay(proj[:, self.a_off:], self.w_a2, self.b_a2, self.tau, decay)
        o = ws.get("gla.o", (t, self.vw), torch.float32)
        ops.gla_scan(proj, self.q_off, self.k_off, self.v_off, decay, self.dk ** -0.5, cache.state, ctx.cu_tokens, ctx.state_slots,
                     ctx.slot_of_token, o, ctx.num_seqs, self.heads, self.dk, self.dv, narrow=ctx.max_query_len > 16)
        y = ws.get("gla.y", (t, self.vw), rt.dtype)
        ops.gla_output(o, proj[:, self.g_off:self.g_off + self.vw], self.norm, self.eps, y, self.heads, self.dv)
        delta = ws.get("mixer.delta_f32", (t, self.hidden), torch.float32)
        return ops.linear(y, self.w_o, None, delta)
