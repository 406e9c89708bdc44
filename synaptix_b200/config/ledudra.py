"""Typed configuration of the Ledudra decoder, read from its config.json.

Keys: ``architecture`` ("Ledudra"), ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (the factor of every branch
when it is added into the residual stream) and ``layers`` (a list; each entry has ``type``, the sizes of its mixer under
``mixer`` and its feed-forward under ``mlp`` or ``null``).  Both layer types are grouped-query attention with
``heads``, ``kv_heads``, ``dim`` (queries and keys), ``vdim`` (values), ``scale``, ``mask.size`` (the sliding window;
absent: every earlier key is seen) and ``v_mix`` (values blended with those of the first layer that says so):

* ``attention``: projections with biases, rotation of neighbouring pairs of the first ``rot.dims`` elements at
  ``rot.base`` with the optional stretch ``rot.scaling`` (``factor``, ``original``, ``fast``, ``slow``), scores mixed
  over heads, sigmoid weights with a bias per head, a gate per head;
* ``attention_2``: q/k RMS norm, no rotation, a learned bias per head and distance bucket (``bias_max`` is the distance
  at which the logarithmic buckets end; the number of buckets is the table's own first size, which ``bias_rows``
  may state for a model whose weights are yet to be made), softmax.

Feed-forward: ``mlp.kind`` = ``dense`` with ``ff``.  Every size and constant is taken from here; a key that is required
and missing, or a type or kind that is not known, is an error.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take


@dataclasses.dataclass(frozen=True)
class RotationSpec:
    dims: int
    base: float
    factor: Optional[float] = None       # the four constants of the stretch, or all None
    original: Optional[float] = None
    fast: Optional[float] = None
    slow: Optional[float] = None

    @classmethod
    def from_dict(cls, d, where):
        sc = d.get("scaling")
        kw = {}
        if sc is not None:
            if not isinstance(sc, dict):
                raise ConfigError(f"{where}: 'scaling' must be an object or null")
            kw = {k: take(sc, k, float, where=where + ".scaling") for k in ("factor", "original", "fast", "slow")}
        return cls(dims=take(d, "dims", int, where=where), base=take(d, "base", float, where=where), **kw)

    def to_dict(self):
        d = {"dims": self.dims, "base": self.base}
        if self.factor is not None:
            d["scaling"] = {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}
        return d


@dataclasses.dataclass(frozen=True)
class MixerSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None
    v_mix: bool = False
    rot: Optional[RotationSpec] = None        # type attention
    bias_max: Optional[float] = None          # type attention_2
    bias_rows: Optional[int] = None           # rows of the distance table; None: the tensor's own size

    @classmethod
    def from_dict(cls, d, typ, where):
        mask = d.get("mask") or {}
        rot = d.get("rot")
        if rot is not None and not isinstance(rot, dict):
            raise ConfigError(f"{where}: 'rot' must be an object or null")
        return cls(heads=take(d, "heads", int, where=where), kv_heads=take(d, "kv_heads", int, where=where),
                   dim=take(d, "dim", int, where=where), vdim=take(d, "vdim", int, where=where),
                   scale=take(d, "scale", float, where=where), window=take(mask, "size", int, None, where=where + ".mask"),
                   v_mix=take(d, "v_mix", bool, False, where=where),
                   rot=RotationSpec.from_dict(rot, where + ".rot") if (rot and typ == "attention") else None,
                   bias_max=take(d, "bias_max", float, where=where) if typ == "attention_2" else None,
                   bias_rows=take(d, "bias_rows", int, None, where=where) if typ == "attention_2" else None)

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "v_mix": self.v_mix}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        if self.bias_max is not None:
            d["bias_max"] = self.bias_max
        if self.bias_rows is not None:
            d["bias_rows"] = self.bias_rows
        return d

    def validate(self, where):
        if min(self.heads, self.kv_heads, self.dim, self.vdim) <= 0 or self.heads % self.kv_heads:
            raise ConfigError(f"{where}: heads must be a positive multiple of kv_heads, dim and vdim positive")
        if self.window is not None and self.window <= 0:
            raise ConfigError(f"{where}: mask.size must be > 0")
        if self.rot is not None:
            r = self.rot
            if r.dims % 2 or not (0 < r.dims <= self.dim) or r.base <= 1:
                raise ConfigError(f"{where}: rot.dims must be even and at most dim, rot.base above 1")
            if r.factor is not None and (r.factor <= 0 or r.original <= 0 or r.fast <= 0 or r.slow <= 0):
                raise ConfigError(f"{where}: rot.scaling needs positive factor, original, fast and slow")


LAYER_TYPES = ("attention", "attention_2")


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: MixerSpec
    ff: Optional[int] = None              # None: the layer has no feed-forward
    ff_kind: Optional[str] = None

    @classmethod
    def from_dict(cls, d, i):
        where = f"config.json: layers[{i}]"
        if not isinstance(d, dict):
            raise ConfigError(f"{where} must be an object")
        typ = take(d, "type", str, where=where)
        if typ not in LAYER_TYPES:
            raise ConfigError(f"{where}: unknown layer type {typ!r} (known: {', '.join(LAYER_TYPES)})")
        mixer = d.get("mixer")
        if not isinstance(mixer, dict):
            raise ConfigError(f"{where}: 'mixer' must be an object")
        kw: Dict[str, Any] = {}
        mlp = d.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict):
                raise ConfigError(f"{where}: 'mlp' must be an object or null")
            kw["ff_kind"] = take(mlp, "kind", str, where=where + ".mlp")
            if kw["ff_kind"] != "dense":
                raise ConfigError(f"{where}.mlp: unknown kind {kw['ff_kind']!r} (known: dense)")
            kw["ff"] = take(mlp, "ff", int, where=where + ".mlp")
        return cls(type=typ, mixer=MixerSpec.from_dict(mixer, typ, where + ".mixer"), **kw)

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.ff is None else {"kind": self.ff_kind, "ff": self.ff}}

    def validate(self, i):
        where = f"config.json: layers[{i}]"
        self.mixer.validate(where + ".mixer")
        if self.type == "attention_2" and (self.mixer.bias_max is None or self.mixer.bias_max <= 0):
            raise ConfigError(f"{where}.mixer: bias_max must be > 0")
        if self.mixer.bias_rows is not None and self.mixer.bias_rows < 2:
            raise ConfigError(f"{where}.mixer: bias_rows must be at least 2")
        if self.ff is not None and self.ff <= 0:
            raise ConfigError(f"{where}.mlp: ff must be > 0")


@dataclasses.dataclass(frozen=True)
class LedudraConfig(ModelConfig):
    architectures: ClassVar[Tuple[str, ...]] = ("Ledudra",)
    model_types: ClassVar[Tuple[str, ...]] = ("ledudra",)

    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    residual_mult: float = 1.0
    layers: Tuple[LayerSpec, ...] = ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LedudraConfig":
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        cfg = cls(vocab=take(d, "vocab", int), width=take(d, "width", int),
                  norm_eps=take(norm, "eps", float, where="config.json: norm"),
                  residual_mult=take(d, "residual_mult", float, 1.0),
                  layers=tuple(LayerSpec.from_dict(x, i) for i, x in enumerate(layers)))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architectures[0], "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                "layers": [x.to_dict() for x in self.layers]}

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: vocab and width must be > 0")
        if self.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        shared = None
        for i, layer in enumerate(self.layers):
            layer.validate(i)
            if layer.mixer.v_mix:
                size = (layer.mixer.kv_heads, layer.mixer.vdim)
                if shared is not None and size != shared:
                    raise ConfigError(f"config.json: layers[{i}] blends its values with the first v_mix layer's, which "
                                      f"has {shared[0]} kv heads of {shared[1]}, not {size[0]} of {size[1]}")
                shared = size

    def first_value_layer(self) -> Optional[int]:
        """The first layer whose values the other ``v_mix`` layers blend theirs with."""
        for i, layer in enumerate(self.layers):
            if layer.mixer.v_mix:
                return i
        return None
