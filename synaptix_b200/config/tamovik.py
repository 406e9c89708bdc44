"""Typed configuration of the Tamovik decoder, read from its config.json.

Keys: ``architecture`` ("Tamovik"), ``vocab``, ``width``, ``norm.eps``, ``embedding.bigram`` (``buckets``, ``mul_prev``,
``mul_cur``: the hashed table of token pairs added to the embedding) and ``layers`` (a list; each entry has ``type``, the
sizes of its mixer under ``mixer`` and its feed-forward under ``mlp`` or ``null``).  Layer types:

* ``latent_attention``: ``heads``, ``dim`` (unrotated query/key elements a head), ``rot_dim`` (rotated ones, the key's
  shared by all heads), ``vdim``, ``kv_rank``, ``scale``, and ``rot`` (``dims``, ``base`` and optionally ``scaling`` with
  ``factor``, ``original``, ``fast``, ``slow``; absent: no rotation);
* ``parallel``: ``left`` (attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` taps, ``scale``, ``mask.size``
  for chunks, absent: every earlier key is seen) and ``right`` (matrix memory: ``heads``, ``dim``, ``vdim``, ``gate_cap``).

Feed-forward: ``mlp.kind`` = ``dense`` with ``ff``, or ``moe`` with ``expert.ff``, ``expert.limit``, ``router.experts``,
``router.top`` and optionally ``router.groups`` (``count``, ``keep``).  Every size and constant is taken from here; a key
that is required and missing, or a type or kind that is not known, is an error.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take


def _obj(d, key, where, required=True):
    v = d.get(key)
    if v is None and not required:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: '{key}' must be an object")
    return v


@dataclasses.dataclass(frozen=True)
class RotationSpec:
    dims: int
    base: float
    factor: Optional[float] = None      # the four numbers of the stretched rotation come together or not at all
    original: Optional[float] = None
    fast: Optional[float] = None
    slow: Optional[float] = None

    @classmethod
    def from_dict(cls, d, where):
        sc = _obj(d, "scaling", where, required=False)
        kw = {}
        if sc is not None:
            kw = {k: take(sc, k, float, where=where + ".scaling") for k in ("factor", "original", "fast", "slow")}
        return cls(dims=take(d, "dims", int, where=where), base=take(d, "base", float, where=where), **kw)

    def to_dict(self):
        d = {"dims": self.dims, "base": self.base}
        if self.factor is not None:
            d["scaling"] = {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}
        return d


@dataclasses.dataclass(frozen=True)
class LatentSpec:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Optional[RotationSpec]

    @classmethod
    def from_dict(cls, d, where):
        rot = _obj(d, "rot", where, required=False)
        return cls(heads=take(d, "heads", int, where=where), dim=take(d, "dim", int, where=where),
                   rot_dim=take(d, "rot_dim", int, where=where), vdim=take(d, "vdim", int, where=where),
                   kv_rank=take(d, "kv_rank", int, where=where), scale=take(d, "scale", float, where=where),
                   rot=None if rot is None else RotationSpec.from_dict(rot, where + ".rot"))

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d

    def validate(self, where):
        if min(self.heads, self.vdim, self.kv_rank) <= 0 or self.dim < 0 or self.rot_dim < 0 or self.dim + self.rot_dim <= 0:
            raise ConfigError(f"{where}: heads, vdim and kv_rank must be > 0, dim + rot_dim > 0")
        r = self.rot
        if r is not None:
            if r.dims % 2 or not (0 < r.dims <= self.rot_dim) or r.base <= 0:
                raise ConfigError(f"{where}: rot.dims must be even and at most rot_dim, rot.base positive")
            if r.factor is not None and (r.factor <= 0 or r.original <= 0 or r.fast <= 0 or r.slow <= 0 or r.base == 1.0):
                raise ConfigError(f"{where}: rot.scaling needs positive numbers")


@dataclasses.dataclass(frozen=True)
class ConvAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    chunk: Optional[int]

    @classmethod
    def from_dict(cls, d, where):
        mask = d.get("mask") or {}
        return cls(heads=take(d, "heads", int, where=where), kv_heads=take(d, "kv_heads", int, where=where),
                   dim=take(d, "dim", int, where=where), vdim=take(d, "vdim", int, where=where),
                   conv=take(d, "conv", int, where=where), scale=take(d, "scale", float, where=where),
                   chunk=take(mask, "size", int, None, where=where + ".mask"))

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv,
             "scale": self.scale}
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        return d

    def validate(self, where):
        if min(self.heads, self.kv_heads, self.dim, self.conv) <= 0 or self.heads % self.kv_heads:
            raise ConfigError(f"{where}: heads, kv_heads, dim and conv must be > 0, heads a multiple of kv_heads")
        if self.vdim != self.dim:
            raise ConfigError(f"{where}: the values are the keys, so vdim must equal dim")
        if self.chunk is not None and self.chunk <= 0:
            raise ConfigError(f"{where}: mask.size must be > 0")


@dataclasses.dataclass(frozen=True)
class MemorySpec:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, d, where):
        return cls(heads=take(d, "heads", int, where=where), dim=take(d, "dim", int, where=where),
                   vdim=take(d, "vdim", int, where=where), gate_cap=take(d, "gate_cap", float, where=where))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}

    def validate(self, where):
        if min(self.heads, self.dim, self.vdim) <= 0 or self.gate_cap <= 0:
            raise ConfigError(f"{where}: heads, dim, vdim and gate_cap must be > 0")


@dataclasses.dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                            # "dense" or "moe"
    ff: int
    limit: Optional[float] = None        # moe: the experts' cap
    experts: int = 0
    top: int = 0
    groups: Optional[Tuple[int, int]] = None     # (count, keep)

    @classmethod
    def from_dict(cls, d, where):
        kind = take(d, "kind", str, where=where)
        if kind == "dense":
            return cls(kind=kind, ff=take(d, "ff", int, where=where))
        if kind != "moe":
            raise ConfigError(f"{where}: unknown kind {kind!r} (known: dense, moe)")
        expert, router = _obj(d, "expert", where), _obj(d, "router", where)
        g = _obj(router, "groups", where + ".router", required=False)
        groups = None if g is None else (take(g, "count", int, where=where + ".router.groups"),
                                         take(g, "keep", int, where=where + ".router.groups"))
        return cls(kind=kind, ff=take(expert, "ff", int, where=where + ".expert"),
                   limit=take(expert, "limit", float, where=where + ".expert"),
                   experts=take(router, "experts", int, where=where + ".router"),
                   top=take(router, "top", int, where=where + ".router"), groups=groups)

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top}
        if self.groups is not None:
            router["groups"] = {"count": self.groups[0], "keep": self.groups[1]}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": router}

    def validate(self, where):
        if self.ff <= 0:
            raise ConfigError(f"{where}: ff must be > 0")
        if self.kind == "moe":
            if not (0 < self.top <= self.experts) or self.limit is None or self.limit <= 0:
                raise ConfigError(f"{where}: 0 < router.top <= router.experts and expert.limit > 0")
            if self.groups is not None:
                count, keep = self.groups
                if count <= 0 or self.experts % count or not (0 < keep <= count) or self.top > keep * (self.experts // count):
                    raise ConfigError(f"{where}: router.groups: equal groups, 0 < keep <= count, and router.top experts "
                                      "must fit the kept groups")


@dataclasses.dataclass(frozen=True)
class TamovikLayer:
    type: str
    latent: Optional[LatentSpec] = None
    left: Optional[ConvAttentionSpec] = None
    right: Optional[MemorySpec] = None
    mlp: Optional[FeedForwardSpec] = None            # None: the layer has no feed-forward

    @classmethod
    def from_dict(cls, d, i):
        where = f"config.json: layers[{i}]"
        if not isinstance(d, dict):
            raise ConfigError(f"{where} must be an object")
        typ = take(d, "type", str, where=where)
        mixer = _obj(d, "mixer", where)
        kw: Dict[str, Any] = {}
        if typ == "latent_attention":
            kw["latent"] = LatentSpec.from_dict(mixer, where + ".mixer")
        elif typ == "parallel":
            kw["left"] = ConvAttentionSpec.from_dict(_obj(mixer, "left", where + ".mixer"), where + ".mixer.left")
            kw["right"] = MemorySpec.from_dict(_obj(mixer, "right", where + ".mixer"), where + ".mixer.right")
        else:
            raise ConfigError(f"{where}: unknown layer type {typ!r} (known: latent_attention, parallel)")
        mlp = _obj(d, "mlp", where, required=False)
        if mlp is not None:
            kw["mlp"] = FeedForwardSpec.from_dict(mlp, where + ".mlp")
        return cls(type=typ, **kw)

    def to_dict(self):
        mixer = self.latent.to_dict() if self.type == "latent_attention" else {"left": self.left.to_dict(),
                                                                              "right": self.right.to_dict()}
        return {"type": self.type, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclasses.dataclass(frozen=True)
class TamovikConfig(ModelConfig):
    architectures: ClassVar[Tuple[str, ...]] = ("Tamovik",)
    model_types: ClassVar[Tuple[str, ...]] = ("tamovik",)

    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    bigram_buckets: int = 0
    bigram_mul_prev: int = 0
    bigram_mul_cur: int = 0
    layers: Tuple[TamovikLayer, ...] = ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TamovikConfig":
        norm = _obj(d, "norm", "config.json")
        big = _obj(_obj(d, "embedding", "config.json"), "bigram", "config.json: embedding")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        w = "config.json: embedding.bigram"
        cfg = cls(vocab=take(d, "vocab", int), width=take(d, "width", int),
                  norm_eps=take(norm, "eps", float, where="config.json: norm"),
                  bigram_buckets=take(big, "buckets", int, where=w), bigram_mul_prev=take(big, "mul_prev", int, where=w),
                  bigram_mul_cur=take(big, "mul_cur", int, where=w),
                  layers=tuple(TamovikLayer.from_dict(x, i) for i, x in enumerate(layers)))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architectures[0], "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps},
                "embedding": {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev,
                                         "mul_cur": self.bigram_mul_cur}},
                "layers": [x.to_dict() for x in self.layers]}

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: vocab and width must be > 0")
        if self.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        if self.bigram_buckets <= 0 or self.bigram_mul_prev < 0 or self.bigram_mul_cur < 0:
            raise ConfigError("config.json: embedding.bigram needs buckets > 0 and multipliers >= 0")
        for i, layer in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            if layer.type == "latent_attention":
                layer.latent.validate(where + ".mixer")
            else:
                layer.left.validate(where + ".mixer.left")
                layer.right.validate(where + ".mixer.right")
            if layer.mlp is not None:
                layer.mlp.validate(where + ".mlp")
