"""FegizenConfig: the keys of a Fegizen config.json, typed.

The file is nested: `vocab`, `width`, `embedding.scale`, `norm.eps`, `canon.taps` (taps of the convolution over time
in front of every sublayer), `logit_scale`, and a list `layers` whose entries give the layer's `type` (its mixer:
'latent_attention', 'gla' or 'gla_2'), the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`: kind
'dense' or 'moe', or null for none).  Every layer has its own sizes.  A latent-attention mixer may name an earlier
layer whose cached latents it reads (`kv_from`).  Field names are the file's keys; `to_dict` writes the same nesting
back.  The width of the middle of a linear-attention mixer's decay map is no key of the file (the tensors' shapes
give it); `decay_rank` is an optional key that the random-weights mode reads.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import BadValue, ConfigReader, WrongArchitecture, read_config_json

ARCHITECTURE = "Fegizen"
LINEAR_ATTENTION_TYPES = ("gla", "gla_2")


@dataclass(frozen=True)
class StretchConfig:
    """`rot.scaling`: how the slow rotary frequencies are lengthened."""
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self) -> dict:
        return dict(factor=self.factor, original=self.original, fast=self.fast, slow=self.slow)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                 # unrotated query/key size of a head
    rot_dim: int             # rotated query/key size of a head (the key's part is shared by all heads)
    vdim: int                # value size of a head
    kv_rank: int             # size of the cached latent
    q_rank: int              # size of the query's latent
    window: int              # mask.size: keys a query sees, itself included (0: no mask in the file, all earlier keys)
    rot_base: float
    rot_dims: int            # rotated dimensions of the rotated part (even, at most rot_dim)
    scale: float
    stretch: Optional[StretchConfig] = None
    kv_from: Optional[int] = None

    @classmethod
    def from_reader(cls, r: ConfigReader, where: str) -> "LatentAttentionConfig":
        rot_dim = r.integer("rot_dim", minimum=0)
        rot = r.section("rot", where=where)
        dims = rot.integer("dims", default=rot_dim, minimum=0)
        if dims % 2 or dims > rot_dim:
            raise BadValue(f"{where}.rot.dims", dims, f"must be even and at most rot_dim = {rot_dim}")
        sc = rot.section("scaling", default=None, where=where + ".rot")
        stretch = None
        if sc is not None:
            stretch = StretchConfig(factor=sc.number("factor", positive=True), original=sc.number("original", positive=True),
                                    fast=sc.number("fast", positive=True), slow=sc.number("slow", positive=True))
        mask = r.section("mask", default=None, where=where)
        dim = r.integer("dim", minimum=1)
        return cls(heads=r.integer("heads", minimum=1), dim=dim, rot_dim=rot_dim,
                   vdim=r.integer("vdim", default=dim, minimum=1), kv_rank=r.integer("kv_rank", minimum=1),
                   q_rank=r.integer("q_rank", minimum=1), window=mask.integer("size", minimum=1) if mask is not None else 0,
                   rot_base=rot.number("base", positive=True), rot_dims=dims, scale=r.number("scale", positive=True),
                   stretch=stretch, kv_from=r.integer("kv_from", default=None, minimum=0))

    def to_dict(self) -> dict:
        rot = dict(base=self.rot_base, dims=self.rot_dims)
        if self.stretch is not None:
            rot["scaling"] = self.stretch.to_dict()
        d = dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, kv_rank=self.kv_rank,
                 q_rank=self.q_rank, rot=rot, scale=self.scale)
        if self.window:
            d["mask"] = dict(size=self.window)
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class LinearAttentionConfig:
    heads: int
    dim: int                 # key size of a head
    vdim: int                # value size of a head
    tau: float               # decays are sigmoid(z)^(1/tau)
    decay_rank: int = 16     # the middle of the decay's map, for the random-weights mode only

    @classmethod
    def from_reader(cls, r: ConfigReader, where: str) -> "LinearAttentionConfig":
        dim = r.integer("dim", minimum=1)
        return cls(heads=r.integer("heads", minimum=1), dim=dim, vdim=r.integer("vdim", default=dim, minimum=1),
                   tau=r.number("tau", positive=True), decay_rank=r.integer("decay_rank", default=16, minimum=1))

    def to_dict(self) -> dict:
        return dict(heads=self.heads, dim=self.dim, vdim=self.vdim, tau=self.tau, decay_rank=self.decay_rank)


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    kind: str = "dense"

    def to_dict(self) -> dict:
        return dict(kind=self.kind, ff=self.ff)


@dataclass(frozen=True)
class RoutedMlpConfig:
    """`mlp` of kind 'moe': `router.experts` experts of inner size `expert.ff` and `router.identity` experts without
    weights, of which a token uses `router.top`; shares are multiplied by `router.scale`; `shared.ff` is the inner
    size of the expert every token uses (None: there is none)."""
    experts: int
    top: int
    ff: int
    identity: int = 0
    scale: float = 1.0
    shared_ff: Optional[int] = None
    kind: str = "moe"

    @classmethod
    def from_reader(cls, r: ConfigReader, where: str) -> "RoutedMlpConfig":
        router = r.section("router", where=where)
        experts = router.integer("experts", minimum=1)
        identity = router.integer("identity", default=0, minimum=0)
        top = router.integer("top", minimum=1)
        if top > experts + identity:
            raise BadValue(f"{where}.router.top", top, f"is more than the {experts + identity} experts")
        shared = r.section("shared", default=None, where=where)
        return cls(experts=experts, top=top, ff=r.section("expert", where=where).integer("ff", minimum=1),
                   identity=identity, scale=router.number("scale", default=1.0),
                   shared_ff=shared.integer("ff", minimum=1) if shared is not None else None)

    def to_dict(self) -> dict:
        d = dict(kind=self.kind, router=dict(experts=self.experts, identity=self.identity, top=self.top, scale=self.scale),
                 expert=dict(ff=self.ff))
        if self.shared_ff is not None:
            d["shared"] = dict(ff=self.shared_ff)
        return d


@dataclass(frozen=True)
class FegizenLayer:
    type: str
    mixer: object            # LatentAttentionConfig or LinearAttentionConfig
    mlp: object              # DenseMlpConfig, RoutedMlpConfig or None

    def to_dict(self) -> dict:
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp else None)


@dataclass(frozen=True)
class FegizenConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    canon_taps: int
    logit_scale: float
    layers: tuple                       # of FegizenLayer

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: dict) -> "FegizenConfig":
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
            if kind == "latent_attention":
                mixer = LatentAttentionConfig.from_reader(m, where + ".mixer")
                src = mixer.kv_from
                if src is not None:
                    if not src < i or layers[src].type != "latent_attention" or layers[src].mixer.kv_from is not None:
                        raise BadValue(f"{where}.mixer.kv_from", src, "must name an earlier latent-attention layer "
                                                                      "that forms latents of its own")
                    own = layers[src].mixer
                    if (own.kv_rank, own.rot_dim, own.rot_base, own.rot_dims, own.stretch) != \
                            (mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims, mixer.stretch):
                        raise BadValue(f"{where}.mixer.kv_from", src, "that layer's latent size or rotation is another one")
            elif kind in LINEAR_ATTENTION_TYPES:
                mixer = LinearAttentionConfig.from_reader(m, where + ".mixer")
            else:
                raise BadValue(f"{where}.type", kind, "known mixers: latent_attention, " + ", ".join(LINEAR_ATTENTION_TYPES))
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
            layers.append(FegizenLayer(type=kind, mixer=mixer, mlp=mlp))
        canon = r.section("canon", default=None)
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   embedding_scale=r.section("embedding").number("scale"),
                   norm_eps=r.section("norm").number("eps", positive=True),
                   canon_taps=canon.integer("taps", minimum=1) if canon is not None else 0,
                   logit_scale=r.number("logit_scale", default=1.0), layers=tuple(layers))

    @classmethod
    def from_json(cls, folder_or_file) -> "FegizenConfig":
        return cls.from_dict(read_config_json(folder_or_file))

    def to_dict(self) -> dict:
        d = dict(architecture=ARCHITECTURE, embedding=dict(scale=self.embedding_scale),
                 layers=[l.to_dict() for l in self.layers], logit_scale=self.logit_scale, norm=dict(eps=self.norm_eps),
                 vocab=self.vocab, width=self.width)
        if self.canon_taps:
            d["canon"] = dict(taps=self.canon_taps)
        return d
