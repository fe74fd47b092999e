"""NodepelConfig: the keys of a Nodepel config.json, typed.

The file is nested: `embedding.scale`, `norm.eps`, `vocab`, `width`, a list `layers` whose entries give the layer's
`type` (its mixer), the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null for none), and
`loop` (`start`, `stop`, `times`: layers start .. stop-1 run `times` times in a row on the same weights, each pass
with a cache and a state of its own).  A mixer of type 'parallel' holds two sides, `left` (softmax attention under a
sliding window with a sink) and `right` (a gated delta rule).  Every layer has its own sizes, so two layers of one
model may differ in all of them.  Field names are the file's keys; `to_dict` writes the same nesting back.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import BadValue, ConfigReader, WrongArchitecture, read_config_json
from .zedivik import LoopConfig

ARCHITECTURE = "Nodepel"


@dataclass(frozen=True)
class SinkAttentionConfig:
    """`mixer.left`: grouped-query attention under a sliding window, rotary positions on part of a head."""
    heads: int
    kv_heads: int
    dim: int                 # query/key size of a head
    vdim: int                # value size of a head
    window: int              # mask.size: keys a query sees, itself included
    rot_base: float
    rot_dims: int            # rotated dimensions of a head (even, at most dim)
    scale: float

    @classmethod
    def from_reader(cls, r: ConfigReader, where: str) -> "SinkAttentionConfig":
        heads = r.integer("heads", minimum=1)
        kv_heads = r.integer("kv_heads", default=heads, minimum=1)
        if heads % kv_heads:
            raise BadValue(f"{where}.kv_heads", kv_heads, f"must divide heads = {heads}")
        dim = r.integer("dim", minimum=1)
        rot = r.section("rot", where=where)
        dims = rot.integer("dims", minimum=0)
        if dims % 2 or dims > dim:
            raise BadValue(f"{where}.rot.dims", dims, f"must be even and at most dim = {dim}")
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=r.integer("vdim", default=dim, minimum=1),
                   window=r.section("mask", where=where).integer("size", minimum=1),
                   rot_base=rot.number("base", positive=True), rot_dims=dims, scale=r.number("scale", positive=True))

    def to_dict(self) -> dict:
        return dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                    mask=dict(size=self.window), rot=dict(base=self.rot_base, dims=self.rot_dims), scale=self.scale)


@dataclass(frozen=True)
class GatedDeltaConfig:
    """`mixer.right`: the gated delta rule."""
    heads: int               # value heads (one state matrix each)
    kv_heads: int            # query/key heads
    dim: int                 # query/key size of a head
    vdim: int                # value size of a head
    conv: int                # taps of the short convolution

    @classmethod
    def from_reader(cls, r: ConfigReader, where: str) -> "GatedDeltaConfig":
        heads = r.integer("heads", minimum=1)
        kv_heads = r.integer("kv_heads", default=heads, minimum=1)
        if heads % kv_heads:
            raise BadValue(f"{where}.kv_heads", kv_heads, f"must divide heads = {heads}")
        dim = r.integer("dim", minimum=1)
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=r.integer("vdim", default=dim, minimum=1),
                   conv=r.integer("conv", minimum=1))

    def to_dict(self) -> dict:
        return dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, conv=self.conv)


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SinkAttentionConfig
    right: GatedDeltaConfig

    def to_dict(self) -> dict:
        return dict(left=self.left.to_dict(), right=self.right.to_dict())


@dataclass(frozen=True)
class MoeConfig:
    """`mlp` of kind 'moe': `router.experts` experts of inner size `expert.ff`, of which a token uses `router.top`;
    `shared.ff` is the inner size of the expert every token uses (None: there is none)."""
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int] = None
    kind: str = "moe"

    @classmethod
    def from_reader(cls, r: ConfigReader, where: str) -> "MoeConfig":
        kind = r.string("kind", default="moe")
        if kind != "moe":
            raise BadValue(f"{where}.kind", kind, "this architecture has routed feed-forwards ('moe') only")
        router = r.section("router", where=where)
        experts = router.integer("experts", minimum=1)
        top = router.integer("top", minimum=1)
        if top > experts:
            raise BadValue(f"{where}.router.top", top, f"is more than the {experts} experts")
        shared = r.section("shared", default=None, where=where)
        return cls(experts=experts, top=top, ff=r.section("expert", where=where).integer("ff", minimum=1),
                   shared_ff=shared.integer("ff", minimum=1) if shared is not None else None, kind=kind)

    def to_dict(self) -> dict:
        d = dict(kind=self.kind, router=dict(experts=self.experts, top=self.top), expert=dict(ff=self.ff))
        if self.shared_ff is not None:
            d["shared"] = dict(ff=self.shared_ff)
        return d


@dataclass(frozen=True)
class NodepelLayer:
    type: str
    mixer: ParallelMixerConfig
    mlp: Optional[MoeConfig]

    def to_dict(self) -> dict:
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp else None)


@dataclass(frozen=True)
class NodepelConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple                       # of NodepelLayer
    loop: Optional[LoopConfig] = None

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: dict) -> "NodepelConfig":
        r = ConfigReader(raw)
        if r.architecture() != ARCHITECTURE:
            raise WrongArchitecture(raw.get("architecture", raw.get("architectures")), ARCHITECTURE)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise BadValue("layers", layers_raw, "must be a non-empty list of layer objects")
        layers = []
        for i, lr in enumerate(layers_raw):
            L = ConfigReader(lr)
            where = f"layers[{i}]"
            kind = L.string("type")
            if kind != "parallel":
                raise BadValue(f"{where}.type", kind, "known mixers: parallel")
            m = L.section("mixer", where=where)
            mixer = ParallelMixerConfig(
                left=SinkAttentionConfig.from_reader(m.section("left", where=where + ".mixer"), where + ".mixer.left"),
                right=GatedDeltaConfig.from_reader(m.section("right", where=where + ".mixer"), where + ".mixer.right"))
            mlp = L.section("mlp", default=None, where=where)
            layers.append(NodepelLayer(type=kind, mixer=mixer,
                                       mlp=MoeConfig.from_reader(mlp, where + ".mlp") if mlp is not None else None))
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
    def from_json(cls, folder_or_file) -> "NodepelConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    def to_dict(self) -> dict:
        d = dict(architecture=ARCHITECTURE, embedding=dict(scale=self.embedding_scale),
                 layers=[l.to_dict() for l in self.layers], norm=dict(eps=self.norm_eps), vocab=self.vocab,
                 width=self.width)
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        return d
