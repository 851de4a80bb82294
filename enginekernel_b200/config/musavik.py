"""Configuration of the Musavik decoder (``"architecture": "Musavik"``).

A Musavik ``config.json`` is nested: ``vocab``, ``width``, ``norm.eps``, ``embedding`` (``scale`` and an
optional ``bigram`` table of hashed token pairs: ``buckets``, ``mul_prev``, ``mul_cur``), an optional ``loop``
(``start``, ``stop``, ``times``) and a list ``layers`` whose entries name their mixer (``type``: ``rglru`` or
``parallel``), the mixer's sizes and constants (``mixer``) and the feed-forward (``mlp`` with ``kind``
``dense``, or null for a layer without one).  A ``parallel`` mixer holds a ``left`` record (attention), a
``right`` record (delta rule) and the two scales of their sum.  Every size and every constant that can
differ between two models of the design is read from the file; nothing is filled in that the file does
not give.
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
            raise ConfigError(f"config.json lacks the required key {where}.{name} for Musavik")
        return default
    return _coerce(f"{where}.{name}", raw[name], kind)


def _positive(obj, names, where):
    for name in names:
        if not getattr(obj, name) > 0:
            raise ConfigError(f"{where}.{name} must be positive, got {getattr(obj, name)}")


@dataclasses.dataclass(frozen=True)
class RglruConfig:
    """``layers[i].mixer`` of an ``rglru`` layer: a gated linear recurrence of ``width`` channels whose two
    gates are block-diagonal products of ``blocks`` equal parts, behind a convolution of ``conv`` taps."""
    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, raw, where):
        g = lambda n: _get(raw, n, int, where)
        return cls(width=g("width"), blocks=g("blocks"), conv=g("conv"))

    def to_dict(self):
        return dataclasses.asdict(self)

    def validate(self, where):
        _positive(self, ("width", "blocks", "conv"), where)
        if self.width % self.blocks:
            raise ConfigError(f"{where}: blocks {self.blocks} does not divide width {self.width}")


@dataclasses.dataclass(frozen=True)
class MixedAttentionConfig:
    """``mixer.left`` of a ``parallel`` layer."""
    heads: int
    kv_heads: int
    dim: int                     # query / key size per head
    vdim: int                    # value size per head
    scale: float
    rot_dims: int                # 0: no rotation
    rot_base: float
    window: Optional[int]        # None: every earlier token is seen
    keep_first: int

    @classmethod
    def from_dict(cls, raw, where):
        g = lambda n, k=int: _get(raw, n, k, where)
        rot = raw.get("rot") if isinstance(raw, dict) else None
        dims, base = 0, 0.0
        if rot is not None:
            dims, base = _get(rot, "dims", int, where + ".rot"), _get(rot, "base", float, where + ".rot")
        mask = raw.get("mask") if isinstance(raw, dict) else None
        window, keep = None, 0
        if mask is not None:
            window = _get(mask, "size", int, where + ".mask", None)
            keep = _get(mask, "keep_first", int, where + ".mask", 0)
        return cls(heads=g("heads"), kv_heads=g("kv_heads"), dim=g("dim"), vdim=g("vdim"), scale=g("scale", float),
                   rot_dims=dims, rot_base=float(base), window=window, keep_first=keep)

    def to_dict(self):
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.window is not None:
            out["mask"] = {"keep_first": self.keep_first, "size": self.window}
        return out

    def validate(self, where):
        _positive(self, ("heads", "kv_heads", "dim", "vdim"), where)
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
class HeadDeltaConfig:
    """``mixer.right`` of a ``parallel`` layer: the delta rule with one decay per head."""
    heads: int                   # value heads
    kv_heads: int                # query / key heads
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, raw, where):
        g = lambda n: _get(raw, n, int, where)
        return cls(heads=g("heads"), kv_heads=g("kv_heads"), dim=g("dim"), vdim=g("vdim"), conv=g("conv"))

    def to_dict(self):
        return dataclasses.asdict(self)

    def validate(self, where):
        _positive(self, ("heads", "kv_heads", "dim", "vdim", "conv"), where)
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}: heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")


@dataclasses.dataclass(frozen=True)
class SideBySideConfig:
    """``layers[i].mixer`` of a ``parallel`` layer: left_scale * left(h) + right_scale * right(h)."""
    left: MixedAttentionConfig
    right: HeadDeltaConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, raw, where):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where} must be a JSON object, got {type(raw).__name__}")
        for side in ("left", "right"):
            if not isinstance(raw.get(side), dict):
                raise ConfigError(f"config.json lacks the required record {where}.{side} for Musavik")
        return cls(left=MixedAttentionConfig.from_dict(raw["left"], where + ".left"),
                   right=HeadDeltaConfig.from_dict(raw["right"], where + ".right"),
                   left_scale=_get(raw, "left_scale", float, where), right_scale=_get(raw, "right_scale", float, where))

    def to_dict(self):
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}

    def validate(self, where):
        self.left.validate(where + ".left")
        self.right.validate(where + ".right")


@dataclasses.dataclass(frozen=True)
class DenseConfig:
    """``layers[i].mlp``: down(gelu_tanh(up(x))), both products with a bias."""
    ff: int
    kind: str = "dense"

    @classmethod
    def from_dict(cls, raw, where):
        kind = _get(raw, "kind", str, where)
        if kind != "dense":
            raise ConfigError(f"{where}.kind is {kind!r}; Musavik has the feed-forward kind 'dense'")
        return cls(ff=_get(raw, "ff", int, where), kind=kind)

    def to_dict(self):
        return {"ff": self.ff, "kind": self.kind}

    def validate(self, where):
        _positive(self, ("ff",), where)


MIXER_TYPES = {"rglru": RglruConfig, "parallel": SideBySideConfig}


@dataclasses.dataclass(frozen=True)
class MusavikLayer:
    type: str
    mixer: Union[RglruConfig, SideBySideConfig]
    mlp: Optional[DenseConfig]

    @classmethod
    def from_dict(cls, raw, where):
        kind = _get(raw, "type", str, where)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"{where}.type is {kind!r}; Musavik has the mixers {', '.join(sorted(MIXER_TYPES))}")
        if "mixer" not in raw or raw["mixer"] is None:
            raise ConfigError(f"config.json lacks the required key {where}.mixer for Musavik")
        mixer = MIXER_TYPES[kind].from_dict(raw["mixer"], where + ".mixer")
        mlp = None if raw.get("mlp") is None else DenseConfig.from_dict(raw["mlp"], where + ".mlp")
        return cls(type=kind, mixer=mixer, mlp=mlp)

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclasses.dataclass(frozen=True)
class PairTableConfig:
    """``embedding.bigram``: row (previous * mul_prev + current * mul_cur) mod buckets of a table with
    buckets + 1 rows is added to a token's embedding; the last row serves a sequence's first token."""
    buckets: int
    mul_prev: int
    mul_cur: int

    @classmethod
    def from_dict(cls, raw, where):
        g = lambda n: _get(raw, n, int, where)
        return cls(buckets=g("buckets"), mul_prev=g("mul_prev"), mul_cur=g("mul_cur"))

    def to_dict(self):
        return dataclasses.asdict(self)


@dataclasses.dataclass(frozen=True)
class LoopConfig:
    """Layers ``start`` .. ``stop - 1`` run ``times`` times in a row with the same weights."""
    start: int
    stop: int
    times: int

    @classmethod
    def from_dict(cls, raw, where):
        g = lambda n: _get(raw, n, int, where)
        return cls(start=g("start"), stop=g("stop"), times=g("times"))

    def to_dict(self):
        return dataclasses.asdict(self)


@dataclasses.dataclass(frozen=True)
class MusavikConfig(ModelConfig):
    architecture = "Musavik"

    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    pair_table: Optional[PairTableConfig] = None
    layers: Tuple[MusavikLayer, ...] = ()
    loop: Optional[LoopConfig] = None

    @classmethod
    def from_dict(cls, raw: dict) -> "MusavikConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config must be a JSON object, got {type(raw).__name__}")
        top = "config.json"
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json lacks the required record 'norm' for Musavik")
        emb = raw.get("embedding")
        if not isinstance(emb, dict):
            raise ConfigError("config.json lacks the required record 'embedding' for Musavik")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json needs a non-empty list 'layers' for Musavik")
        pair = None if emb.get("bigram") is None else PairTableConfig.from_dict(emb["bigram"], "embedding.bigram")
        loop = None if raw.get("loop") is None else LoopConfig.from_dict(raw["loop"], "loop")
        cfg = cls(vocab=_get(raw, "vocab", int, top), width=_get(raw, "width", int, top),
                  norm_eps=_get(norm, "eps", float, "norm"), embedding_scale=_get(emb, "scale", float, "embedding"),
                  pair_table=pair,
                  layers=tuple(MusavikLayer.from_dict(l, f"layers[{i}]") for i, l in enumerate(layers)), loop=loop)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        _positive(self, ("vocab", "width", "norm_eps"), "config.json")
        if not self.layers:
            raise ConfigError("Musavik needs at least one layer")
        for i, layer in enumerate(self.layers):
            layer.mixer.validate(f"layers[{i}].mixer")
            if layer.mlp is not None:
                layer.mlp.validate(f"layers[{i}].mlp")
        if self.pair_table is not None:
            _positive(self.pair_table, ("buckets",), "embedding.bigram")
            if self.pair_table.mul_prev < 0 or self.pair_table.mul_cur < 0:
                raise ConfigError("embedding.bigram: the multipliers cannot be negative")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start < lp.stop <= len(self.layers)) or lp.times < 1:
                raise ConfigError(f"loop: start {lp.start}, stop {lp.stop}, times {lp.times} do not name a stretch "
                                  f"of the {len(self.layers)} layers run at least once")

    def to_dict(self) -> dict:
        emb = {"scale": self.embedding_scale}
        if self.pair_table is not None:
            emb["bigram"] = self.pair_table.to_dict()
        out = {"architecture": self.architecture, "embedding": emb, "layers": [l.to_dict() for l in self.layers],
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            out["loop"] = self.loop.to_dict()
        return out

    def runs(self):
        """(layer, pass or None, starts a pass) in execution order: the layers before the loop once, the
        stretch ``times`` times, the rest once."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None, False) for i in range(n)]
        lp = self.loop
        out = [(i, None, False) for i in range(lp.start)]
        for p in range(lp.times):
            out += [(i, p, i == lp.start) for i in range(lp.start, lp.stop)]
        return out + [(i, None, False) for i in range(lp.stop, n)]
