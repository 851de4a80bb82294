"""Configuration of the Bolelix decoder (``"architecture": "Bolelix"``).

A Bolelix ``config.json`` is nested: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and a list
``layers`` whose entries name their mixer (``type``: ``attention``, ``mamba2`` or ``mlstm``), the mixer's
sizes and constants (``mixer``) and the feed-forward (``mlp``: routed experts, ``kind`` ``moe``, or null for
a layer without one).  An attention layer may name another layer whose keys and values it reads
(``kv_from``).  Every size and every constant that can differ between two models of the design is read
from the file; nothing is filled in that the file does not give.
"""

from __future__ import annotations

import dataclasses
from typing import Optional, Tuple, Union

from .base import ConfigError, ModelConfig, _coerce


def _get(raw, name, kind, where, default=dataclasses.MISSING):
    if not isinstance(raw, dict):
        raise ConfigError(f"{where} must be a JSON object, got {type(raw).__name__}")
    if name not in raw or raw[name] is None:
        if default is dataclasses.MISSING:
            raise ConfigError(f"config.json lacks the required key {where}.{name} for Bolelix")
        return default
    return _coerce(f"{where}.{name}", raw[name], kind)


def _positive(obj, names, where):
    for name in names:
        if not getattr(obj, name) > 0:
            raise ConfigError(f"{where}.{name} must be positive, got {getattr(obj, name)}")


@dataclasses.dataclass(frozen=True)
class WindowAttentionConfig:
    """``layers[i].mixer`` of an ``attention`` layer."""
    heads: int
    kv_heads: int
    dim: int                     # query / key size per head
    vdim: int                    # value size per head
    scale: float
    rot_dims: int                # 0: no rotation
    rot_base: float
    rot_factor: float            # every frequency is divided by it (1: plain)
    window: Optional[int]        # None: every earlier token is seen
    keep_first: int
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, raw, where):
        g = lambda n, k=int: _get(raw, n, k, where)
        rot = raw.get("rot") if isinstance(raw, dict) else None
        dims = base = 0
        factor = 1.0
        if rot is not None:
            dims, base = _get(rot, "dims", int, where + ".rot"), _get(rot, "base", float, where + ".rot")
            scaling = rot.get("scaling")
            if scaling is not None:
                factor = _get(scaling, "factor", float, where + ".rot.scaling")
        mask = raw.get("mask") if isinstance(raw, dict) else None
        window, keep = None, 0
        if mask is not None:
            window = _get(mask, "size", int, where + ".mask", None)
            keep = _get(mask, "keep_first", int, where + ".mask", 0)
        return cls(heads=g("heads"), kv_heads=g("kv_heads"), dim=g("dim"), vdim=g("vdim"), scale=g("scale", float),
                   rot_dims=dims, rot_base=float(base), rot_factor=factor, window=window, keep_first=keep,
                   kv_from=_get(raw, "kv_from", int, where, None))

    def to_dict(self):
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_factor != 1.0:
                out["rot"]["scaling"] = {"factor": self.rot_factor}
        if self.window is not None:
            out["mask"] = {"keep_first": self.keep_first, "size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out

    def validate(self, where):
        _positive(self, ("heads", "kv_heads", "dim", "vdim", "rot_factor"), where)
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}: heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        if self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ConfigError(f"{where}: rot.dims {self.rot_dims} must be even and at most dim {self.dim}")
        if self.rot_dims and not self.rot_base > 0:
            raise ConfigError(f"{where}: rot.base must be positive")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"{where}: mask.size must be at least 1")
        if self.keep_first < 0 or (self.keep_first and self.window is None):
            raise ConfigError(f"{where}: mask.keep_first needs mask.size and cannot be negative")


@dataclasses.dataclass(frozen=True)
class Mamba2Config:
    """``layers[i].mixer`` of a ``mamba2`` layer."""
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, raw, where):
        g = lambda n: _get(raw, n, int, where)
        return cls(heads=g("heads"), vdim=g("vdim"), state=g("state"), groups=g("groups"), conv=g("conv"),
                   norm_groups=g("norm_groups"))

    def to_dict(self):
        return dataclasses.asdict(self)

    def validate(self, where):
        _positive(self, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), where)
        if self.heads % self.groups:
            raise ConfigError(f"{where}: heads {self.heads} is not a multiple of groups {self.groups}")
        if (self.heads * self.vdim) % self.norm_groups:
            raise ConfigError(f"{where}: norm_groups {self.norm_groups} does not divide heads * vdim")


@dataclasses.dataclass(frozen=True)
class MlstmConfig:
    """``layers[i].mixer`` of an ``mlstm`` layer."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, raw, where):
        g = lambda n, k=int: _get(raw, n, k, where)
        return cls(heads=g("heads"), dim=g("dim"), vdim=g("vdim"), gate_cap=g("gate_cap", float))

    def to_dict(self):
        return dataclasses.asdict(self)

    def validate(self, where):
        _positive(self, ("heads", "dim", "vdim", "gate_cap"), where)


@dataclasses.dataclass(frozen=True)
class ExpertsConfig:
    """``layers[i].mlp``: routed experts."""
    ff: int                  # of one expert
    experts: int
    top: int
    kind: str = "moe"

    @classmethod
    def from_dict(cls, raw, where):
        kind = _get(raw, "kind", str, where)
        if kind != "moe":
            raise ConfigError(f"{where}.kind {kind!r} is not a Bolelix feed-forward (moe)")
        router = raw.get("router")
        return cls(ff=_get(raw.get("expert"), "ff", int, where + ".expert"),
                   experts=_get(router, "experts", int, where + ".router"),
                   top=_get(router, "top", int, where + ".router"))

    def to_dict(self):
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}

    def validate(self, where):
        _positive(self, ("ff", "experts", "top"), where)
        if self.top > self.experts:
            raise ConfigError(f"{where}.router: top {self.top} exceeds the {self.experts} experts")


@dataclasses.dataclass(frozen=True)
class BolelixLayer:
    type: str
    mixer: Union[WindowAttentionConfig, Mamba2Config, MlstmConfig]
    mlp: Optional[ExpertsConfig]

    MIXERS = {"attention": WindowAttentionConfig, "mamba2": Mamba2Config, "mlstm": MlstmConfig}

    @classmethod
    def from_dict(cls, raw, where):
        kind = _get(raw, "type", str, where)
        if kind not in cls.MIXERS:
            raise ConfigError(f"{where}.type {kind!r} is not a Bolelix mixer ({', '.join(cls.MIXERS)})")
        if raw.get("mixer") is None:
            raise ConfigError(f"config.json lacks the required key {where}.mixer for Bolelix")
        mlp = raw.get("mlp")
        return cls(kind, cls.MIXERS[kind].from_dict(raw["mixer"], where + ".mixer"),
                   None if mlp is None else ExpertsConfig.from_dict(mlp, where + ".mlp"))

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclasses.dataclass(frozen=True)
class BolelixConfig(ModelConfig):
    architecture = "Bolelix"

    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    layers: Tuple[BolelixLayer, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "BolelixConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config must be a JSON object, got {type(raw).__name__}")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError('config.json needs "layers": a list with one entry per layer')
        cfg = cls(vocab=_get(raw, "vocab", int, "config"), width=_get(raw, "width", int, "config"),
                  norm_eps=_get(raw.get("norm"), "eps", float, "norm"),
                  embedding_scale=_get(raw.get("embedding") or {}, "scale", float, "embedding", 1.0),
                  layers=tuple(BolelixLayer.from_dict(l, f"layers[{i}]") for i, l in enumerate(layers)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab", "width"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if not self.layers:
            raise ConfigError("a Bolelix model needs at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}].mixer"
            layer.mixer.validate(where)
            if layer.mlp is not None:
                layer.mlp.validate(f"layers[{i}].mlp")
            src = getattr(layer.mixer, "kv_from", None)
            if src is None:
                continue
            if not 0 <= src < i or self.layers[src].type != "attention" or self.layers[src].mixer.kv_from is not None:
                raise ConfigError(f"{where}.kv_from {src} must name an earlier attention layer with keys and "
                                  "values of its own")
            mine, theirs = layer.mixer, self.layers[src].mixer
            if (mine.kv_heads, mine.dim, mine.vdim) != (theirs.kv_heads, theirs.dim, theirs.vdim):
                raise ConfigError(f"{where}: kv_heads, dim and vdim must equal those of layer {src}, whose keys "
                                  "and values it reads")

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                "layers": [l.to_dict() for l in self.layers], "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width}
