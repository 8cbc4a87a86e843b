"""Attention whose keys and values are made from one latent vector per token: only the latent and one rotated key
part, shared by all heads, are kept in the cache."""
from __future__ import annotations

import torch

from .. import ops
from . import wide_attend
from ..weights.loader import TensorDecl
from .base import POSITION_ENCODINGS, CachePlane, Mixer, PagedCache, matrix, register_mixer, vector_f32


@register_mixer("latent_attention")
class LatentAttention(wide_attend.WideAttendPlan, Mixer):
    """x -> q = Wq x, head by head [dn unrotated | dr rotated];  Wdkv x = [latent (r) | key part (dr)].
    c = latent / rms(latent) * w (eps inside the root); kr = the key part, rotated, shared by all heads.
    Per head h: k_h = Wuk_h c (dn), v_h = Wuv_h c (dv); score = scale * (q_plain . k_h + q_rot . kr) over the keys the
    window lets the row see; plain softmax; the heads' values side by side are multiplied by sigmoid(Wg x) and go
    through the output projection.

    The cache holds one plane of r + dr numbers per token, [c | kr].  Keys and values are never made: since
    q_plain . (Wuk_h c) = (Wuk_h^T q_plain) . c, the query is carried into the latent's coordinates, the attention
    runs with ONE key/value head of r + dr key and r value coordinates (both read from the same plane) for all
    query heads, and Wuv_h is applied to the attended latent.  Norm, rotation (the position encoding's table), scores
    and softmax are float32, and so are the carried query and the gate; the delta is float32.

    params: prefix, hidden_size, num_heads, plain_dim (dn), rotated_dim (dr), value_dim (dv), latent_dim (r), scale, eps,
    window (or None), gate (False: no output gate), position (a PartSpec of a rotary encoding over the dr coordinates, or
    None).  Tensors under the prefix: q, dkv, dkv.norm, uk [heads*dn, r], uv [heads*dv, r], g, o.
    """

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden, self.heads = int(spec["hidden_size"]), int(spec["num_heads"])
        self.dn, self.dr, self.dv, self.r = int(spec["plain_dim"]), int(spec["rotated_dim"]), int(spec["value_dim"]), int(spec["latent_dim"])
        if self.r > 512:
            raise ValueError(f"latent_attention: a latent of {self.r} coordinates is more than the kernel covers (512)")
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.window = spec.get("window")
        self.has_gate = bool(spec.get("gate", True))
        self.position = POSITION_ENCODINGS.build(spec["position"]) if spec.get("position") is not None else None
        self.qw, self.kvw, self.ow = self.heads * (self.dn + self.dr), self.r + self.dr, self.heads * self.dv

    def cache_need(self):
        return PagedCache((CachePlane("latent", 1, self.kvw),), self.window)

    def tensors(self):
        p = self.prefix
        out = [
            TensorDecl(p + "q", (self.qw, self.hidden)), TensorDecl(p + "dkv", (self.kvw, self.hidden)),
            TensorDecl(p + "dkv.norm", (self.r,), init="scale"), TensorDecl(p + "uk", (self.heads * self.dn, self.r)),
            TensorDecl(p + "uv", (self.ow, self.r)), TensorDecl(p + "o", (self.hidden, self.ow)),
        ]
        if self.has_gate:
            out.append(TensorDecl(p + "g", (self.ow, self.hidden)))
        if self.position is not None:
            out += self.position.tensors()
        return out

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        inputs = [tensors[p + "q"], tensors[p + "dkv"]] + ([tensors[p + "g"]] if self.has_gate else [])
        self.w_in = matrix(torch.cat(inputs, dim=0), rt)
        # per head: the keys' up-projection transposed ([r, dn]: carries a query into the latent's coordinates) and the
        # values' up-projection as it is ([dv, r])
        self.w_uk_t = matrix(tensors[p + "uk"].reshape(self.heads, self.dn, self.r).transpose(1, 2), rt)
        self.w_uv = matrix(tensors[p + "uv"].reshape(self.heads, self.dv, self.r), rt)
        self.w_o = matrix(tensors[p + "o"], rt)
        self.latent_norm = vector_f32(tensors[p + "dkv.norm"])
        self.fast = wide_attend.supports(rt, self.kvw, self.r, self.kvw, False)  # bfloat16: the tensor-core kernel
        self.table, self.rot = None, 0
        if self.position is not None:
            self.position.bind(tensors, rt)
            self.table = self.position.rotary_table(rt)
            if self.table is None or not self.position.interleaved:
                raise ValueError("latent_attention: the position encoding must be a rotary one with interleaved pairs")
            self.rot = self.position.rotary_dim
            self.graph_safe = bool(self.position.graph_safe)

    def forward(self, ctx, x, cache, owns_cache=True):
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        h, r, wide = self.heads, self.r, self.kvw
        proj = ws.get("latent_attn.in", (t, self.w_in.shape[0]), torch.float32)
        ops.linear(x, self.w_in, None, proj)
        q_wide = ws.get("latent_attn.q_wide", (t, h, wide), torch.float32)
        q_plain = ws.get("latent_attn.q_plain", (t, h, self.dn), rt.dtype)
        pages, table = cache.planes["latent"], cache.block_table(ctx)
        ops.latent_encode(proj, self.qw, self.latent_norm, self.eps, self.table, self.rot, ctx.positions, ctx.slot_of_token, table,
                          q_wide, q_plain, pages, h, self.dn, self.dr, r, store=owns_cache)
        ops.linear_heads(q_plain, self.w_uk_t, q_wide[:, :, :r])
        attended = ws.get("latent_attn.attended", (t, h, r), rt.dtype)
        wide_attend.attend(ctx, rt, self.fast, table, q_wide.view(t, h * wide), pages, pages, attended.view(t, h * r), None, h, 1, wide, r,
                           self.window, self.scale)
        values = ws.get("latent_attn.values", (t, h, self.dv), torch.float32)
        ops.linear_heads(attended, self.w_uv, values)
        if self.has_gate:
            gated = ws.get("latent_attn.gated", (t, self.ow), rt.dtype)
            ops.sigmoid_gate_mul(values.view(t, self.ow), proj[:, self.qw + self.kvw:], gated)
        elif rt.dtype == torch.float32:
            gated = values.view(t, self.ow)
        else:
            gated = ws.get("latent_attn.gated", (t, self.ow), rt.dtype).copy_(values.view(t, self.ow))
        delta = ws.get("mixer.delta_f32", (t, self.hidden), torch.float32)
        return ops.linear(gated, self.w_o, None, delta)
