"""TubepelConfig: the keys of a Tubepel config.json, typed.

The file is nested: `vocab`, `width`, `norm.eps`, `streams` (copies of the residual stream that every sublayer reads
from and writes to through learned weights; absent or null: one plain residual stream), `loop` (start, stop, times:
the stretch of layers that runs several times in a row; absent or null: none), and a list `layers` whose entries
give the layer's `type` (its mixer: 'latent_attention', 'latent_attention_2' or 'attention'), the mixer's sizes and
constants (`mixer`) and its feed-forward (`mlp`: kind 'dense' or 'moe', or null for none).  Every layer has its own
sizes.  Field names are the file's keys; `to_dict` writes the same nesting back.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import BadValue, ConfigReader, WrongArchitecture, read_config_json

ARCHITECTURE = "Tubepel"
# which dimensions of a rotated vector form a pair, by the mixer's type name
LATENT_PAIRING = {"latent_attention": "neighbours", "latent_attention_2": "halves"}


def _rotation(r: ConfigReader, where: str, size: int, whole: bool):
    """(base, dims) of a `rot` section: dims even and at most `size`; `whole` wants dims == size."""
    rot = r.section("rot", default=None, where=where)
    if rot is None:
        return 10000.0, 0
    dims = rot.integer("dims", default=size, minimum=0)
    if dims % 2 or dims > size or (whole and dims != size):
        raise BadValue(f"{where}.rot.dims", dims, f"must be even and {'equal to' if whole else 'at most'} {size}")
    return rot.number("base", positive=True), dims


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                 # unrotated query/key size of a head
    rot_dim: int             # rotated query/key size of a head (the key's part is shared by all heads)
    vdim: int                # value size of a head
    kv_rank: int             # size of the cached latent
    q_rank: int              # size of the query's latent
    rot_base: float
    rot_dims: int            # = rot_dim: the whole rotated part turns
    scale: float

    @classmethod
    def from_reader(cls, r: ConfigReader, where: str) -> "LatentAttentionConfig":
        rot_dim = r.integer("rot_dim", minimum=0)
        base, dims = _rotation(r, where, rot_dim, whole=True)
        dim = r.integer("dim", minimum=1)
        return cls(heads=r.integer("heads", minimum=1), dim=dim, rot_dim=rot_dim,
                   vdim=r.integer("vdim", default=dim, minimum=1), kv_rank=r.integer("kv_rank", minimum=1),
                   q_rank=r.integer("q_rank", minimum=1), rot_base=base, rot_dims=dims,
                   scale=r.number("scale", positive=True))

    def to_dict(self) -> dict:
        return dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, kv_rank=self.kv_rank,
                    q_rank=self.q_rank, rot=dict(base=self.rot_base, dims=self.rot_dims), scale=self.scale)


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int                 # query/key size of a head
    vdim: int                # value size of a head
    window: int              # mask.size: the last keys a query sees, itself included (0: no mask, all earlier keys)
    keep_first: int          # mask.keep_first: the first keys of a request stay visible behind the window
    rot_base: float
    rot_dims: int            # rotated dimensions of a head (even, at most dim; 0: none)
    scale: float

    @classmethod
    def from_reader(cls, r: ConfigReader, where: str) -> "WindowAttentionConfig":
        heads, dim = r.integer("heads", minimum=1), r.integer("dim", minimum=1)
        kv_heads = r.integer("kv_heads", default=heads, minimum=1)
        if heads % kv_heads:
            raise BadValue(f"{where}.kv_heads", kv_heads, f"must divide the {heads} query heads")
        base, dims = _rotation(r, where, dim, whole=False)
        mask = r.section("mask", default=None, where=where)
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=r.integer("vdim", default=dim, minimum=1),
                   window=mask.integer("size", minimum=1) if mask is not None else 0,
                   keep_first=mask.integer("keep_first", default=0, minimum=0) if mask is not None else 0,
                   rot_base=base, rot_dims=dims, scale=r.number("scale", positive=True))

    def to_dict(self) -> dict:
        d = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                 rot=dict(base=self.rot_base, dims=self.rot_dims), scale=self.scale)
        if self.window:
            d["mask"] = dict(size=self.window, keep_first=self.keep_first)
        return d


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    kind: str = "dense"

    def to_dict(self) -> dict:
        return dict(kind=self.kind, ff=self.ff)


@dataclass(frozen=True)
class RoutedMlpConfig:
    """`mlp` of kind 'moe': `router.experts` experts of inner size `expert.ff` of which a token uses `router.top`;
    `shared.ff` is the inner size of the expert every token uses (None: there is none)."""
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int] = None
    kind: str = "moe"

    @classmethod
    def from_reader(cls, r: ConfigReader, where: str) -> "RoutedMlpConfig":
        router = r.section("router", where=where)
        experts = router.integer("experts", minimum=1)
        top = router.integer("top", minimum=1)
        if top > experts:
            raise BadValue(f"{where}.router.top", top, f"is more than the {experts} experts")
        shared = r.section("shared", default=None, where=where)
        return cls(experts=experts, top=top, ff=r.section("expert", where=where).integer("ff", minimum=1),
                   shared_ff=shared.integer("ff", minimum=1) if shared is not None else None)

    def to_dict(self) -> dict:
        d = dict(kind=self.kind, router=dict(experts=self.experts, top=self.top), expert=dict(ff=self.ff))
        if self.shared_ff is not None:
            d["shared"] = dict(ff=self.shared_ff)
        return d


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int

    def to_dict(self) -> dict:
        return dict(start=self.start, stop=self.stop, times=self.times)


@dataclass(frozen=True)
class TubepelLayer:
    type: str
    mixer: object            # LatentAttentionConfig or WindowAttentionConfig
    mlp: object              # DenseMlpConfig, RoutedMlpConfig or None

    def to_dict(self) -> dict:
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp else None)


@dataclass(frozen=True)
class TubepelConfig:
    vocab: int
    width: int
    norm_eps: float
    streams: int                        # 0: one plain residual stream
    loop: Optional[LoopConfig]
    layers: tuple                       # of TubepelLayer

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: dict) -> "TubepelConfig":
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
            m = L.section("mixer", where=where)
            if kind in LATENT_PAIRING:
                mixer = LatentAttentionConfig.from_reader(m, where + ".mixer")
            elif kind == "attention":
                mixer = WindowAttentionConfig.from_reader(m, where + ".mixer")
            else:
                raise BadValue(f"{where}.type", kind, "known mixers: attention, " + ", ".join(LATENT_PAIRING))
            mlp = None
            mr = L.section("mlp", default=None, where=where)
            if mr is not None:
                mk = mr.string("kind")
                if mk == "dense":
                    mlp = DenseMlpConfig(ff=mr.integer("ff", minimum=1))
                elif mk == "moe":
                    mlp = RoutedMlpConfig.from_reader(mr, where + ".mlp")
                else:
                    raise BadValue(f"{where}.mlp.kind", mk, "known feed-forwards: dense, moe")
            layers.append(TubepelLayer(type=kind, mixer=mixer, mlp=mlp))
        loop = None
        lp = r.section("loop", default=None)
        if lp is not None:
            loop = LoopConfig(start=lp.integer("start", minimum=0), stop=lp.integer("stop", minimum=0),
                              times=lp.integer("times", minimum=1))
            if not loop.start <= loop.stop <= len(layers):
                raise BadValue("loop", lp.raw, f"needs start <= stop <= {len(layers)} layers")
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   norm_eps=r.section("norm").number("eps", positive=True),
                   streams=r.integer("streams", default=0, minimum=0), loop=loop, layers=tuple(layers))

    @classmethod
    def from_json(cls, folder_or_file) -> "TubepelConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    def to_dict(self) -> dict:
        d = dict(architecture=ARCHITECTURE, layers=[l.to_dict() for l in self.layers], norm=dict(eps=self.norm_eps),
                 vocab=self.vocab, width=self.width)
        if self.streams:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        return d
