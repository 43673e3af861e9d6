"""Typed configuration of the Mugedra decoder, read from its config.json.

Keys: `architecture` ("Mugedra"), `vocab`, `width`, `norm.eps`, optional `loop` (`start`, `stop`, `times`: the
layers start .. stop - 1 run `times` times in a row with the same tensors and a cache or state per pass), and
`layers`: a list whose entries give `type` ("parallel"), the mixer's sizes and constants under `mixer` and the
feed-forward under `mlp` (null: none; `kind` "moe" with `expert.ff`, `router.experts`, `router.top`).

parallel mixer: two branches that read the same input.
`left` (softmax attention): `heads`, `kv_heads`, `dim`, `vdim`, `scale`, optional `softcap`, optional `mask.size`
(a query sees the keys of its own chunk of that many positions), optional `rot` (`dims`, `base`, optional `scaling`
with `factor`, `original`, `fast`, `slow`).
`right` (gated delta rule): `heads`, `kv_heads`, `dim`, `vdim`, `conv` (taps of the short convolution).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader

ARCHITECTURE = "Mugedra"
MAX_POSITIONS = 131072      # the design names no longest sequence; rotation tables are made for as many positions as an engine allows, at most this


def _object(data: Any, where: str) -> Dict[str, Any]:
    if not isinstance(data, dict):
        raise ConfigError(f"key '{where}' must be an object, got {data!r}")
    return data


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]] = None     # factor, original, fast, slow

    def to_dict(self):
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return d


@dataclass(frozen=True)
class ChunkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0               # 0: scores are not capped
    chunk: int = 0                     # mask.size; 0: every earlier key is seen
    rot: Optional[RotaryConfig] = None

    def to_dict(self):
        d: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                             "vdim": self.vdim}
        if self.softcap:
            d["softcap"] = self.softcap
        if self.chunk:
            d["mask"] = {"size": self.chunk}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class DeltaRuleConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                          # taps

    def to_dict(self):
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: ChunkAttentionConfig
    right: DeltaRuleConfig

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class MoeConfig:
    ff: int
    experts: int
    top: int

    def to_dict(self):
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class MugedraLayer:
    type: str                                   # "parallel"
    mixer: ParallelMixerConfig
    mlp: Optional[MoeConfig]

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int

    def to_dict(self):
        return {"start": self.start, "stop": self.stop, "times": self.times}


def _heads(r: KeyReader, where: str) -> Tuple[int, int]:
    heads, kv_heads = r.integer("heads"), r.integer("kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"key '{where}.heads' ({heads}) must be divisible by 'kv_heads' ({kv_heads})")
    return heads, kv_heads


def _read_left(raw: Dict[str, Any], where: str) -> ChunkAttentionConfig:
    r = KeyReader(raw)
    heads, kv_heads = _heads(r, where)
    dim = r.integer("dim")
    chunk = 0
    if raw.get("mask") is not None and _object(raw["mask"], where + ".mask").get("size") is not None:
        chunk = KeyReader(raw["mask"]).integer("size")
    rot = None
    if raw.get("rot") is not None:
        rr = _object(raw["rot"], where + ".rot")
        k = KeyReader(rr)
        dims = k.integer("dims")
        if dims % 2 or dims > dim:
            raise ConfigError(f"key '{where}.rot.dims' must be even and at most 'dim' ({dim}), got {dims}")
        scaling = None
        if rr.get("scaling") is not None:
            s = KeyReader(_object(rr["scaling"], where + ".rot.scaling"))
            scaling = (s.number("factor"), s.number("original"), s.number("fast"), s.number("slow"))
        rot = RotaryConfig(dims, k.number("base"), scaling)
    return ChunkAttentionConfig(heads, kv_heads, dim, r.integer("vdim"), r.number("scale"),
                                softcap=r.number("softcap", 0.0, positive=False), chunk=chunk, rot=rot)


def _read_right(raw: Dict[str, Any], where: str) -> DeltaRuleConfig:
    r = KeyReader(raw)
    heads, kv_heads = _heads(r, where)
    return DeltaRuleConfig(heads, kv_heads, r.integer("dim"), r.integer("vdim"), r.integer("conv", 1))


@dataclass(frozen=True)
class MugedraConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[MugedraLayer, ...]
    loop: Optional[LoopConfig] = None

    ARCHITECTURE = ARCHITECTURE

    @property
    def max_positions(self) -> int:
        return MAX_POSITIONS

    def stop_token_ids(self) -> Tuple[int, ...]:
        return ()

    def runs(self) -> Tuple[Tuple[int, bool], ...]:
        """(layer, whether the embedding's output joins the residual stream right before it) for every place in
        the order of execution: the layers before the loop, the looped layers once per pass (every pass but the
        first begins with the embedding's output added), the layers after it."""
        n = len(self.layers)
        if self.loop is None:
            return tuple((i, False) for i in range(n))
        lp = self.loop
        out = [(i, False) for i in range(lp.start)]
        for p in range(lp.times):
            out += [(i, p > 0 and i == lp.start) for i in range(lp.start, lp.stop)]
        return tuple(out + [(i, False) for i in range(lp.stop, n)])

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MugedraConfig":
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
            if kind != "parallel":
                raise ConfigError(f"key '{where}.type': unsupported value {kind!r} (supported: 'parallel')")
            mixer_raw = _object(raw.get("mixer"), where + ".mixer")
            mixer = ParallelMixerConfig(
                _read_left(_object(mixer_raw.get("left"), where + ".mixer.left"), where + ".mixer.left"),
                _read_right(_object(mixer_raw.get("right"), where + ".mixer.right"), where + ".mixer.right"))
            mlp = None
            if raw.get("mlp") is not None:
                m = _object(raw["mlp"], where + ".mlp")
                if m.get("kind") != "moe":
                    raise ConfigError(f"key '{where}.mlp.kind': unsupported value {m.get('kind')!r} (supported: 'moe')")
                router = KeyReader(_object(m.get("router"), where + ".mlp.router"))
                experts, top = router.integer("experts"), router.integer("top")
                if top > experts:
                    raise ConfigError(f"key '{where}.mlp.router.top' ({top}) exceeds 'experts' ({experts})")
                mlp = MoeConfig(KeyReader(_object(m.get("expert"), where + ".mlp.expert")).integer("ff"), experts, top)
            layers.append(MugedraLayer(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lr = KeyReader(_object(d["loop"], "loop"))
            loop = LoopConfig(lr.integer("start", minimum=0), lr.integer("stop", minimum=0), lr.integer("times"))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"key 'loop': layers {loop.start} .. {loop.stop} - 1 do not lie within the "
                                  f"{len(layers)} layers")
            if loop.start == loop.stop:
                loop = None
        return cls(vocab=r.integer("vocab"), width=r.integer("width"), eps=norm.number("eps"), layers=tuple(layers),
                   loop=loop)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": ARCHITECTURE, "layers": [layer.to_dict() for layer in self.layers],
                             "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        return d
