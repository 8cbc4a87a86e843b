"""The Fozutar decoder: its config.json keys, typed and checked, and its model as data.

config.json names the design under `architecture` and gives `vocab`, `width`, `max_positions`, `norm.eps`,
`embedding.scale`, the list `layers` and, optionally, `loop`.  Every layer is a parallel one with ONE RMS norm that its
mixer and its feed-forward both read, and names its mixer under `type` with that mixer's sizes under `mixer`:

* `attention`: heads, kv_heads (heads if absent), dim (query/key size per head), vdim, scale, softcap (none if absent),
  bias_max, mask {size} (every earlier key if absent).  Grouped heads
  with q and k biases, the values are the projected keys, every head normed on its own, a soft cap on the scores, a
  learned bias by distance (table `rel`), a mask by chunks of mask.size positions, no rotation.
* `gla`: heads, dim (key channels per head), vdim, tau.  Gated linear attention with a low-rank decay projection.

`mlp` is null, {kind: "dense", ff} (GELU, tanh form) or {kind: "moe", expert {ff}, router {experts, top}} (SiLU experts,
a router with a bias, softmax over the chosen logits).  `loop` {start, stop, times}: layers start..stop-1 run `times`
times in a row with the same weights and a cache or state of their own each time; before every pass but the first the
embedding's output is added to the stream, and before every pass the pass's vector (`loop.step`).

Two sizes are given by tensor shapes alone: the rows of an attention layer's bias table (`rel` [rows, heads]) and the
rank of a gla layer's decay projection (`a1` [rank, width]).  A configuration made from a folder reads them there
(`with_tensor_shapes`); `to_json` writes them as `bias_rows` and `decay_rank`, which `from_json` takes when present,
so that a configuration made in memory (random weights) is whole.

Tensor names: embed, pos, final.norm, loop.step, and per layer i: l<i>.norm1, l<i>.mix.*, l<i>.mlp.*.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import ConfigError, JsonReader, ModelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, RunSpec, part
from .venarax import LayerLoop, _sub


@dataclass(frozen=True)
class ChunkedAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    bias_max: float
    chunk: Optional[int]  # None: every earlier key is visible
    bias_rows: Optional[int] = None  # rows of the bias table: from the tensor `rel` when config.json does not say

    @classmethod
    def read(cls, r: JsonReader) -> "ChunkedAttentionSizes":
        heads = r.integer("heads")
        kv = r.integer("kv_heads", heads)
        if heads % kv:
            raise ConfigError(f"{r.where}: heads {heads} is not a multiple of kv_heads {kv}")
        dim = r.integer("dim")
        vdim = r.integer("vdim", dim)
        if vdim != dim:
            raise ConfigError(f"{r.where}: the values are the keys, so vdim {vdim} must equal dim {dim}")
        mask = _sub(r.raw, "mask", r.where, required=False)
        softcap = r.number("softcap") if r.raw.get("softcap") is not None else None
        return cls(heads, kv, dim, vdim, r.number("scale"), softcap, r.number("bias_max"),
                   mask.integer("size") if mask else None, r.optional_integer("bias_rows", minimum=2))

    def to_json(self) -> Dict[str, Any]:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
               "bias_max": self.bias_max}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        if self.bias_rows is not None:
            out["bias_rows"] = self.bias_rows
        return out

    def missing(self) -> bool:
        return self.bias_rows is None

    def resolved(self, prefix: str, shapes: Mapping[str, Tuple[int, ...]], where: str):
        if self.bias_rows is not None:
            return self
        shape = shapes.get(prefix + "rel")
        if shape is None or len(shape) != 2:
            raise ConfigError(f"{where}: the bias table '{prefix}rel' [rows, heads] is not among the tensors")
        return replace(self, bias_rows=int(shape[0]))


@dataclass(frozen=True)
class GlaSizes:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: Optional[int] = None  # from the tensor `a1` when config.json does not say

    @classmethod
    def read(cls, r: JsonReader) -> "GlaSizes":
        return cls(r.integer("heads"), r.integer("dim"), r.integer("vdim"), r.number("tau"), r.optional_integer("decay_rank"))

    def to_json(self) -> Dict[str, Any]:
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        return out

    def missing(self) -> bool:
        return self.decay_rank is None

    def resolved(self, prefix: str, shapes: Mapping[str, Tuple[int, ...]], where: str):
        if self.decay_rank is not None:
            return self
        shape = shapes.get(prefix + "a1")
        if shape is None or len(shape) != 2:
            raise ConfigError(f"{where}: the decay projection '{prefix}a1' [rank, width] is not among the tensors")
        return replace(self, decay_rank=int(shape[0]))


_MIXERS = {"attention": ChunkedAttentionSizes, "gla": GlaSizes}


@dataclass(frozen=True)
class DenseSizes:
    ff: int

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class MoeSizes:
    ff: int
    experts: int
    top: int

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


def _read_mlp(mlp: Optional[JsonReader]):
    if mlp is None:
        return None
    kind = mlp.string("kind")
    if kind == "dense":
        return DenseSizes(mlp.integer("ff"))
    if kind == "moe":
        expert, router = _sub(mlp.raw, "expert", mlp.where), _sub(mlp.raw, "router", mlp.where)
        experts, top = router.integer("experts"), router.integer("top")
        if top > experts:
            raise ConfigError(f"{router.where}: top {top} is more than the {experts} experts")
        return MoeSizes(expert.integer("ff"), experts, top)
    raise ConfigError(f"{mlp.where}: kind '{kind}' is not supported (dense, moe)")


@dataclass(frozen=True)
class FozutarLayer:
    type: str
    mixer: Any  # ChunkedAttentionSizes or GlaSizes
    mlp: Any  # DenseSizes, MoeSizes or None


@register_architecture("Fozutar")
@dataclass(frozen=True)
class FozutarConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    max_positions: int
    layers: Tuple[FozutarLayer, ...]
    loop: Optional[LayerLoop]

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "FozutarConfig":
        r = JsonReader(raw)
        norm = _sub(raw, "norm", "config.json")
        emb = _sub(raw, "embedding", "config.json", required=False)
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(listed):
            where = f"config.json.layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where}: must be an object")
            kind = JsonReader(entry, where).string("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{where}: type '{kind}' is not a mixer of this design ({', '.join(sorted(_MIXERS))})")
            sizes = _MIXERS[kind].read(_sub(entry, "mixer", where))
            layers.append(FozutarLayer(kind, sizes, _read_mlp(_sub(entry, "mlp", where, required=False))))
        loop = _sub(raw, "loop", "config.json", required=False)
        if loop is not None:
            loop = LayerLoop(loop.integer("start", minimum=0), loop.integer("stop"), loop.integer("times"))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json.loop: layers {loop.start}..{loop.stop - 1} are not a range of the {len(layers)} layers")
        return cls(r.integer("vocab"), r.integer("width"), norm.number("eps"), emb.number("scale") if emb else 1.0,
                   r.integer("max_positions"), tuple(layers), loop)

    def to_json(self) -> Dict[str, Any]:
        out = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
            "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.type, "mixer": l.mixer.to_json(), "mlp": l.mlp.to_json() if l.mlp else None} for l in self.layers],
        }
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    # ------------------------------------------------------------------ sizes that only the tensors give

    def needs_tensor_shapes(self) -> bool:
        return any(l.mixer.missing() for l in self.layers)

    def with_tensor_shapes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "FozutarConfig":
        layers = tuple(replace(l, mixer=l.mixer.resolved(f"l{i}.mix.", shapes, f"config.json.layers[{i}]")) for i, l in enumerate(self.layers))
        return replace(self, layers=layers)

    # ------------------------------------------------------------------ the model as data

    def _norm(self, name: str):
        return part("rmsnorm", tensor=name, size=self.width, eps=self.eps)

    def _mixer(self, layer: FozutarLayer, prefix: str):
        m = layer.mixer
        if m.missing():
            raise ConfigError(f"{prefix}: a size that only the tensors give is not known yet (load the configuration from the "
                              "model's folder, or give bias_rows / decay_rank)")
        if layer.type == "attention":
            return part("chunked_attention", prefix=prefix, hidden_size=self.width, num_heads=m.heads, num_kv_heads=m.kv_heads,
                        key_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=self.eps, bias=True, values_are_keys=True, head_norm=True,
                        softcap=m.softcap, bias_rows=m.bias_rows, bias_reach=m.bias_max, chunk=m.chunk, max_positions=self.max_positions)
        return part("gated_linear_attention", prefix=prefix, hidden_size=self.width, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                    decay_rank=m.decay_rank, tau=m.tau, eps=self.eps)

    def _mlp(self, layer: FozutarLayer, prefix: str):
        m = layer.mlp
        if m is None:
            return None
        if isinstance(m, DenseSizes):
            return part("gated_mlp", prefix=prefix, hidden_size=self.width, intermediate_size=m.ff, activation="gelu_tanh")
        return part("routed_experts", prefix=prefix, hidden_size=self.width, intermediate_size=m.ff, experts=m.experts, top=m.top,
                    activation="silu", router_bias=True)

    def run_order(self) -> Tuple[RunSpec, ...]:
        """Every layer once, except that the looped range runs `times` times in a row: each run has its own cache or state, and
        the first layer of every pass is preceded by the pass's entry."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(RunSpec(i) for i in range(n))
        lp = self.loop
        runs = [RunSpec(i) for i in range(lp.start)]
        for t in range(lp.times):
            entry = part("add_embedding", vectors="loop.step", rows=lp.times, row=t, hidden_size=self.width, add_first=t > 0)
            runs += [RunSpec(i, entry=entry if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return tuple(runs + [RunSpec(i) for i in range(lp.stop, n)])

    def model_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            layers.append(LayerSpec(block="parallel", mixer=self._mixer(layer, p + "mix."), feed_forward=self._mlp(layer, p + "mlp."),
                                    mixer_norm=self._norm(p + "norm1"), feed_forward_norm=None, prefix=p))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=part("scaled_position_embedding", tensor="embed", vocab_size=self.vocab, hidden_size=self.width,
                           scale=self.embedding_scale, positions="pos", max_positions=self.max_positions),
            layers=tuple(layers), run_order=self.run_order(), final_norm=self._norm("final.norm"),
            head=part("lm_head", tensor="head", tied_to="embed", vocab_size=self.vocab, hidden_size=self.width),
            max_positions=self.max_positions,
        )
