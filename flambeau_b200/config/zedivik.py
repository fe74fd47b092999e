"""ZedivikConfig: the keys of a Zedivik config.json, typed.

The file is nested: `embedding.scale`, `norm.eps`, `vocab`, `width`, a list `layers` whose entries give the layer's
`type`, its mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null for none), and `loop`
(`start`, `stop`, `times`: layers start .. stop-1 run `times` times in a row on the same weights, each pass with a
cache of its own).  Every layer has its own sizes, so two layers of one model may differ in all of them.  Field
names are the file's keys; `to_dict` writes the same nesting back.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import BadValue, ConfigReader, WrongArchitecture, read_config_json

ARCHITECTURE = "Zedivik"


@dataclass(frozen=True)
class DiffAttentionConfig:
    """`mixer` of a layer of type 'attention' (differential attention under a sliding window)."""
    heads: int
    kv_heads: int
    dim: int                 # per-map query/key size
    vdim: int                # value size of a head
    window: int              # mask.size: keys a query sees, itself included
    scale: float
    diff: float              # the constant of lambda and of the (1 - diff) output factor

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "DiffAttentionConfig":
        heads = r.integer("heads", minimum=1)
        kv_heads = r.integer("kv_heads", default=heads, minimum=1)
        if heads % kv_heads:
            raise BadValue("kv_heads", kv_heads, f"must divide heads = {heads}")
        mask = r.section("mask", where="mixer")
        return cls(heads=heads, kv_heads=kv_heads, dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1),
                   window=mask.integer("size", minimum=1), scale=r.number("scale", positive=True),
                   diff=r.number("diff"))

    def to_dict(self) -> dict:
        return dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                    mask=dict(size=self.window), scale=self.scale, diff=self.diff)


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    kind: str = "dense"

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "DenseMlpConfig":
        kind = r.string("kind", default="dense")
        if kind != "dense":
            raise BadValue("mlp.kind", kind, "this architecture has dense feed-forwards only")
        return cls(ff=r.integer("ff", minimum=1), kind=kind)

    def to_dict(self) -> dict:
        return dict(ff=self.ff, kind=self.kind)


@dataclass(frozen=True)
class ZedivikLayer:
    type: str
    mixer: DiffAttentionConfig
    mlp: Optional[DenseMlpConfig]

    def to_dict(self) -> dict:
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp else None)


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int

    def to_dict(self) -> dict:
        return dict(start=self.start, stop=self.stop, times=self.times)


@dataclass(frozen=True)
class ZedivikConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple                       # of ZedivikLayer
    loop: Optional[LoopConfig] = None

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: dict) -> "ZedivikConfig":
        r = ConfigReader(raw)
        if r.architecture() != ARCHITECTURE:
            raise WrongArchitecture(raw.get("architecture", raw.get("architectures")), ARCHITECTURE)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise BadValue("layers", layers_raw, "must be a non-empty list of layer objects")
        layers = []
        for i, lr in enumerate(layers_raw):
            L = ConfigReader(lr)
            kind = L.string("type")
            if kind != "attention":
                raise BadValue(f"layers[{i}].type", kind, "known mixers: attention")
            mlp = L.section("mlp", default=None, where=f"layers[{i}]")
            layers.append(ZedivikLayer(type=kind,
                                       mixer=DiffAttentionConfig.from_reader(L.section("mixer", where=f"layers[{i}]")),
                                       mlp=DenseMlpConfig.from_reader(mlp) if mlp is not None else None))
        loop = None
        lp = r.section("loop", default=None)
        if lp is not None:
            loop = LoopConfig(start=lp.integer("start", minimum=0), stop=lp.integer("stop", minimum=0),
                              times=lp.integer("times", minimum=1))
            if not loop.start < loop.stop <= len(layers):
                raise BadValue("loop", loop.to_dict(), f"needs 0 <= start < stop <= {len(layers)} layers")
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   embedding_scale=r.section("embedding").number("scale"),
                   norm_eps=r.section("norm").number("eps", positive=True), layers=tuple(layers), loop=loop)

    @classmethod
    def from_json(cls, folder_or_file) -> "ZedivikConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    def to_dict(self) -> dict:
        d = dict(architecture=ARCHITECTURE, embedding=dict(scale=self.embedding_scale),
                 layers=[l.to_dict() for l in self.layers], norm=dict(eps=self.norm_eps), vocab=self.vocab,
                 width=self.width)
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        return d
