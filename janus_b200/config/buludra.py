"""Typed configuration of the Buludra decoder, read from its config.json.

Keys: `architecture` ("Buludra"), `vocab`, `width`, `norm.eps`, optional `logit_softcap`, and `layers`: a list whose
entries give `type` (which mixer the layer has), the mixer's sizes and constants under `mixer`, the feed-forward under
`mlp` (null: none), and optionally `weights_of`: the index of the layer whose tensors this layer uses (its entry
otherwise equals that layer's; it keeps a cache or state of its own).

type "attention" (softmax attention with normed heads and a query temperature): `heads`, `kv_heads`, `dim`, `vdim`,
`scale`, optional `q_temp` (`coef`, `every`).
type "gla" (gated linear attention): `heads`, `dim`, `vdim`, `tau`; the rank of the decay's projection is the shape
of its tensor, so `rank` is optional here and the model's builder may be told it.
type "parallel": `left` (softmax attention with a sink: `heads`, `kv_heads`, `dim`, `vdim`, `scale`, optional `rot`
with `dims`, `base`), `right` (matrix memory: `heads`, `dim`, `vdim`, `gate_cap`), `left_scale`, `right_scale`.

mlp: `kind` "dense" with `ff`, or "moe" with `expert.ff`, `router.experts`, `router.top`, optional `router.groups`
(`count`, `keep`) and optional `shared` (`ff`).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple, Union

from .base import ConfigError, KeyReader

ARCHITECTURE = "Buludra"
MAX_POSITIONS = 131072      # the design names no longest sequence; rotation tables are made for as many positions as an engine allows, at most this
DEFAULT_DECAY_RANK = 16     # for configurations that are written without a folder of tensors to read the rank from


def _object(data: Any, where: str) -> Dict[str, Any]:
    if not isinstance(data, dict):
        raise ConfigError(f"key '{where}' must be an object, got {data!r}")
    return data


def _heads(r: KeyReader, where: str) -> Tuple[int, int]:
    heads, kv_heads = r.integer("heads"), r.integer("kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"key '{where}.heads' ({heads}) must be divisible by 'kv_heads' ({kv_heads})")
    return heads, kv_heads


@dataclass(frozen=True)
class TemperatureAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float = 0.0
    temp_every: int = 0                 # 0: no query temperature

    def to_dict(self):
        d: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                             "vdim": self.vdim}
        if self.temp_every:
            d["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        return d


@dataclass(frozen=True)
class GlaConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int = DEFAULT_DECAY_RANK

    def to_dict(self):
        return {"dim": self.dim, "heads": self.heads, "rank": self.rank, "tau": self.tau, "vdim": self.vdim}


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int = 0                   # 0: no rotation
    rot_base: float = 10000.0

    def to_dict(self):
        d: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                             "vdim": self.vdim}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    def to_dict(self):
        return {"dim": self.dim, "gate_cap": self.gate_cap, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class SideBySideConfig:
    left: SinkAttentionConfig
    right: MatrixMemoryConfig
    left_scale: float
    right_scale: float

    def to_dict(self):
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class DenseConfig:
    ff: int

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int
    top: int
    groups: int = 0                     # 0: every expert can be chosen
    keep: int = 0
    shared_ff: int = 0                  # 0: no shared expert

    def to_dict(self):
        router: Dict[str, Any] = {"experts": self.experts, "top": self.top}
        if self.groups:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        d: Dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe", "router": router}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


MixerConfig = Union[TemperatureAttentionConfig, GlaConfig, SideBySideConfig]


@dataclass(frozen=True)
class BuludraLayer:
    type: str                                   # "attention", "gla" or "parallel"
    mixer: MixerConfig
    mlp: Union[DenseConfig, ExpertsConfig, None]
    weights_of: Optional[int] = None

    def to_dict(self):
        d: Dict[str, Any] = {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                             "type": self.type}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


def _read_attention(raw: Dict[str, Any], where: str) -> TemperatureAttentionConfig:
    r = KeyReader(raw)
    heads, kv_heads = _heads(r, where)
    coef, every = 0.0, 0
    if raw.get("q_temp") is not None:
        t = KeyReader(_object(raw["q_temp"], where + ".q_temp"))
        coef, every = t.number("coef", positive=False), t.integer("every")
    return TemperatureAttentionConfig(heads, kv_heads, r.integer("dim"), r.integer("vdim"), r.number("scale"), coef, every)


def _read_gla(raw: Dict[str, Any], where: str) -> GlaConfig:
    r = KeyReader(raw)
    return GlaConfig(r.integer("heads"), r.integer("dim"), r.integer("vdim"), r.number("tau"),
                     r.integer("rank", DEFAULT_DECAY_RANK))


def _read_side_by_side(raw: Dict[str, Any], where: str) -> SideBySideConfig:
    lraw = _object(raw.get("left"), where + ".left")
    lr = KeyReader(lraw)
    heads, kv_heads = _heads(lr, where + ".left")
    dim = lr.integer("dim")
    rot_dims, rot_base = 0, 10000.0
    if lraw.get("rot") is not None:
        k = KeyReader(_object(lraw["rot"], where + ".left.rot"))
        rot_dims, rot_base = k.integer("dims"), k.number("base")
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"key '{where}.left.rot.dims' must be even and at most 'dim' ({dim}), got {rot_dims}")
    left = SinkAttentionConfig(heads, kv_heads, dim, lr.integer("vdim"), lr.number("scale"), rot_dims, rot_base)
    rr = KeyReader(_object(raw.get("right"), where + ".right"))
    right = MatrixMemoryConfig(rr.integer("heads"), rr.integer("dim"), rr.integer("vdim"), rr.number("gate_cap"))
    r = KeyReader(raw)
    return SideBySideConfig(left, right, r.number("left_scale", positive=False), r.number("right_scale", positive=False))


_MIXERS = {"attention": _read_attention, "gla": _read_gla, "parallel": _read_side_by_side}


def _read_mlp(raw: Any, where: str):
    if raw is None:
        return None
    m = _object(raw, where)
    kind = m.get("kind")
    if kind == "dense":
        return DenseConfig(KeyReader(m).integer("ff"))
    if kind != "moe":
        raise ConfigError(f"key '{where}.kind': unsupported value {kind!r} (supported: 'dense', 'moe')")
    rraw = _object(m.get("router"), where + ".router")
    router = KeyReader(rraw)
    experts, top = router.integer("experts"), router.integer("top")
    if top > experts:
        raise ConfigError(f"key '{where}.router.top' ({top}) exceeds 'experts' ({experts})")
    groups = keep = 0
    if rraw.get("groups") is not None:
        g = KeyReader(_object(rraw["groups"], where + ".router.groups"))
        groups, keep = g.integer("count"), g.integer("keep")
        if experts % groups or keep > groups or keep * (experts // groups) < top:
            raise ConfigError(f"key '{where}.router.groups': {groups} groups of which {keep} are kept do not fit "
                              f"{experts} experts and {top} a token")
    shared = 0
    if m.get("shared") is not None:
        shared = KeyReader(_object(m["shared"], where + ".shared")).integer("ff")
    return ExpertsConfig(KeyReader(_object(m.get("expert"), where + ".expert")).integer("ff"), experts, top, groups,
                         keep, shared)


@dataclass(frozen=True)
class BuludraConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[BuludraLayer, ...]
    logit_softcap: float = 0.0          # 0: logits are not capped

    ARCHITECTURE = ARCHITECTURE

    @property
    def max_positions(self) -> int:
        return MAX_POSITIONS

    def stop_token_ids(self) -> Tuple[int, ...]:
        return ()

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses (a layer may name one that names another in turn)."""
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
        return i

    def with_tensor_shapes(self, shape_of) -> "BuludraConfig":
        """The configuration with the sizes that only a tensor's shape gives: the rank of a gated-linear-attention
        layer's decay projection is the number of rows of its `mix.a1`.  `shape_of(name)` gives a tensor's shape, or
        None where the folder has no such tensor (the configuration's own value then stands)."""
        layers = list(self.layers)
        for i, layer in enumerate(layers):
            if layer.type == "gla" and layer.weights_of is None:
                shape = shape_of(f"l{i}.mix.a1")
                if shape is not None and len(shape) == 2:
                    layers[i] = replace(layer, mixer=replace(layer.mixer, rank=int(shape[0])))
        for i, layer in enumerate(layers):
            if layer.weights_of is not None:
                layers[i] = replace(layer, mixer=layers[self.owner(i)].mixer)
        return replace(self, layers=tuple(layers))

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "BuludraConfig":
        r = KeyReader(d)
        norm = KeyReader(_object(d.get("norm"), "norm"))
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"key 'layers' must be a non-empty list, got {type(raw_layers).__name__}")
        layers = []
        for i, raw in enumerate(raw_layers):
            where = f"layers[{i}]"
            raw = _object(raw, where)
            kind = raw.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"key '{where}.type': unsupported value {kind!r} (supported: {sorted(_MIXERS)})")
            mixer = _MIXERS[kind](_object(raw.get("mixer"), where + ".mixer"), where + ".mixer")
            weights_of = None
            if raw.get("weights_of") is not None:
                weights_of = KeyReader(raw).integer("weights_of", minimum=0)
            layers.append(BuludraLayer(kind, mixer, _read_mlp(raw.get("mlp"), where + ".mlp"), weights_of))
        for i, layer in enumerate(layers):
            j = layer.weights_of
            if j is None:
                continue
            seen = {i}
            while j is not None and j < len(layers) and j not in seen:      # a chain ends at a layer with tensors
                seen.add(j)
                j, last = layers[j].weights_of, j
            if j is not None:
                raise ConfigError(f"key 'layers[{i}].weights_of' must lead to another layer that has tensors of its own, "
                                  f"got {layer.weights_of}")
            j = last
            if (layers[j].type, layers[j].mixer, layers[j].mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"key 'layers[{i}]': a layer that uses layer {j}'s tensors must have its sizes and constants")
        return cls(vocab=r.integer("vocab"), width=r.integer("width"), eps=norm.number("eps"), layers=tuple(layers),
                   logit_softcap=r.number("logit_softcap", 0.0, positive=False))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": ARCHITECTURE, "layers": [layer.to_dict() for layer in self.layers],
                             "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d
