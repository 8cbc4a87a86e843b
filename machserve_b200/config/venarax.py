"""The Venarax decoder: its config.json keys, typed and checked, and its model as data.

config.json names the design under `architecture`, gives `vocab`, `width`, `norm.eps`, the list `layers` and,
optionally, `loop`.  Every layer is a parallel one (mixer and feed-forward read two layer norms of the same stream)
and names its mixer under `type` with that mixer's sizes under `mixer`:

* `attention`: heads, kv_heads, dim (query/key size per head), vdim (value size per head), scale,
  q_temp {coef, every}.  Grouped heads, norm over the whole query and key projections, no rotation, a sink per head.
* `latent_attention`: heads, dim (unrotated) and rot_dim (rotated query/key sizes per head), vdim, kv_rank (size of
  the cached latent), scale, rot {base, dims}, mask {size} (sliding window).

`mlp` is null or {kind: "dense", ff, limit}.  `loop` {start, stop, times}: layers start..stop-1 run `times` times in a
row with the same weights and a cache of their own each time; every pass begins with the stream mixed with the
embedding's output (`loop.in`) plus the pass's vector (`loop.step`).  The config gives no limit on positions:
the engine's own limit (its cache) stands.

Tensor names: embed, head, final.norm(.b), loop.in, loop.step, and per layer i: l<i>.norm1(.b), l<i>.norm2(.b),
l<i>.mix.*, l<i>.mlp.{gate,up,down}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import ConfigError, JsonReader, ModelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, RunSpec, part

NO_POSITION_LIMIT = 1 << 30


def _sub(raw: Mapping[str, Any], key: str, where: str, required: bool = True) -> Optional[JsonReader]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"{where}: key '{key}' is required")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: '{key}' must be an object, found {v!r}")
    return JsonReader(v, f"{where}.{key}")


@dataclass(frozen=True)
class SinkAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float
    temp_every: int

    @classmethod
    def read(cls, r: JsonReader) -> "SinkAttentionSizes":
        heads, kv = r.integer("heads"), r.integer("kv_heads")
        if heads % kv:
            raise ConfigError(f"{r.where}: heads {heads} is not a multiple of kv_heads {kv}")
        t = _sub(r.raw, "q_temp", r.where, required=False)
        coef = t.number("coef", positive=False) if t else 0.0
        every = t.integer("every") if t else 1
        return cls(heads, kv, r.integer("dim"), r.integer("vdim"), r.number("scale"), coef, every)

    def to_json(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                "q_temp": {"coef": self.temp_coef, "every": self.temp_every}}


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    window: Optional[int]

    @classmethod
    def read(cls, r: JsonReader) -> "LatentAttentionSizes":
        rot = _sub(r.raw, "rot", r.where)
        mask = _sub(r.raw, "mask", r.where, required=False)
        rot_dim, dims = r.integer("rot_dim"), rot.integer("dims")
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"{r.where}: rot.dims {dims} must be even and at most rot_dim {rot_dim}")
        return cls(r.integer("heads"), r.integer("dim"), rot_dim, r.integer("vdim"), r.integer("kv_rank"), r.number("scale"),
                   rot.number("base"), dims, mask.integer("size") if mask else None)

    def to_json(self) -> Dict[str, Any]:
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
               "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


_MIXERS = {"attention": SinkAttentionSizes, "latent_attention": LatentAttentionSizes}


@dataclass(frozen=True)
class DenseMlpSizes:
    ff: int
    limit: float

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class VenaraxLayer:
    type: str
    mixer: Any  # SinkAttentionSizes or LatentAttentionSizes
    mlp: Optional[DenseMlpSizes]


@dataclass(frozen=True)
class LayerLoop:
    start: int
    stop: int
    times: int


@register_architecture("Venarax")
@dataclass(frozen=True)
class VenaraxConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    layers: Tuple[VenaraxLayer, ...]
    loop: Optional[LayerLoop]

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "VenaraxConfig":
        r = JsonReader(raw)
        norm = _sub(raw, "norm", "config.json")
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
            mlp = _sub(entry, "mlp", where, required=False)
            if mlp is not None:
                if mlp.string("kind") != "dense":
                    raise ConfigError(f"{where}.mlp: kind '{mlp.string('kind')}' is not supported (dense)")
                mlp = DenseMlpSizes(mlp.integer("ff"), mlp.number("limit"))
            layers.append(VenaraxLayer(kind, sizes, mlp))
        loop = _sub(raw, "loop", "config.json", required=False)
        if loop is not None:
            loop = LayerLoop(loop.integer("start", minimum=0), loop.integer("stop"), loop.integer("times"))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json.loop: layers {loop.start}..{loop.stop - 1} are not a range of the {len(layers)} layers")
        return cls(r.integer("vocab"), r.integer("width"), norm.number("eps"), tuple(layers), loop)

    def to_json(self) -> Dict[str, Any]:
        out = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
            "layers": [{"type": l.type, "mixer": l.mixer.to_json(), "mlp": l.mlp.to_json() if l.mlp else None} for l in self.layers],
        }
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    # ------------------------------------------------------------------ the model as data

    def _norm(self, name: str):
        return part("layernorm", tensor=name, bias=name + ".b", size=self.width, eps=self.eps)

    def _mixer(self, layer: VenaraxLayer, prefix: str):
        m = layer.mixer
        if layer.type == "attention":
            return part("sink_attention", prefix=prefix, hidden_size=self.width, num_heads=m.heads, num_kv_heads=m.kv_heads,
                        key_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=self.eps, temp_coef=m.temp_coef,
                        temp_every=m.temp_every, window=None, sink=True)
        return part("latent_attention", prefix=prefix, hidden_size=self.width, num_heads=m.heads, plain_dim=m.dim,
                    rotated_dim=m.rot_dim, value_dim=m.vdim, latent_dim=m.kv_rank, scale=m.scale, eps=self.eps, window=m.window,
                    gate=True, position=part("rope", head_dim=m.rot_dim, rotary_dim=m.rot_dims, theta=m.rot_base, pairing="interleaved"))

    def run_order(self) -> Tuple[RunSpec, ...]:
        """Every layer once, except that the looped range runs `times` times in a row: each run has its own cache, and
        the first layer of every pass is preceded by the pass's entry."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(RunSpec(i) for i in range(n))
        lp = self.loop
        runs = [RunSpec(i) for i in range(lp.start)]
        for t in range(lp.times):
            entry = part("mix_with_embedding", matrix="loop.in", vectors="loop.step", rows=lp.times, row=t, hidden_size=self.width)
            runs += [RunSpec(i, entry=entry if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return tuple(runs + [RunSpec(i) for i in range(lp.stop, n)])

    def model_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            ffn = None
            if layer.mlp is not None:
                ffn = part("clamped_glu", prefix=p + "mlp.", hidden_size=self.width, intermediate_size=layer.mlp.ff,
                           limit=layer.mlp.limit, alpha=1.702, shift=1.0)
            layers.append(LayerSpec(block="parallel", mixer=self._mixer(layer, p + "mix."), feed_forward=ffn,
                                    mixer_norm=self._norm(p + "norm1"), feed_forward_norm=self._norm(p + "norm2") if ffn else None,
                                    prefix=p))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=part("embedding", tensor="embed", vocab_size=self.vocab, hidden_size=self.width),
            layers=tuple(layers), run_order=self.run_order(), final_norm=self._norm("final.norm"),
            head=part("lm_head", tensor="head", tied_to=None, vocab_size=self.vocab, hidden_size=self.width),
            max_positions=NO_POSITION_LIMIT,
        )
