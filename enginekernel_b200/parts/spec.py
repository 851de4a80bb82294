"""Plain-data description of a model: which parts, with which sizes, in which order.

An architecture's builder turns its configuration into a :class:`ModelSpec`.
Nothing here holds tensors or launches kernels; the engine instantiates the
registered part classes from it.  The reference has no such layer (its one model
is written out in engine/ek_model.py:280-416); it exists so that layers can differ
from one another and the order of execution is data.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part reads, by its full name in the safetensors files.  A size of
    -1 in ``shape`` is free: the file decides it (the part reads it off the tensor it is handed);
    random weights take ``free_size`` there."""
    name: str
    shape: Tuple[int, ...]
    #: how the random-weights mode fills it: "linear" and "embedding" are N(0, std),
    #: "gain" is 1 + N(0, std_gain); "int" tensors are integer tables
    init: str = "linear"
    #: "float" tensors are computed with in the engine's dtype; "int" become int32
    numeric: str = "float"
    #: another tensor name that may stand in when this one is absent (tied weights)
    optional_alias: Optional[str] = None
    #: what a free size (-1 in ``shape``) becomes when weights are drawn at random
    free_size: int = 16

    def concrete_shape(self) -> Tuple[int, ...]:
        return tuple(self.free_size if d < 0 else d for d in self.shape)

    def fits(self, shape) -> bool:
        shape = tuple(shape)
        return len(shape) == len(self.shape) and all(w < 0 or w == g for w, g in zip(self.shape, shape))


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """A part chosen by ``kind`` with its sizes and constants in ``params``.

    ``weights`` maps the part's own role names (``"q"``, ``"gate"``, ``"gain"``...)
    to checkpoint tensor names, so no part knows the naming of any model.
    """
    kind: str
    params: Dict[str, object] = dataclasses.field(default_factory=dict)
    weights: Dict[str, str] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer, a feed-forward and its norms."""
    block: PartSpec
    mixer: PartSpec
    feed_forward: Optional[PartSpec]        # None: the layer is its mixer alone
    norms: Dict[str, PartSpec]


@dataclasses.dataclass(frozen=True)
class RunSpec:
    """One entry of the execution order.

    ``layer`` indexes :attr:`ModelSpec.layers` (a layer may run more than once).
    ``cache`` names the cache entry its mixer uses; two runs naming the same entry
    share it, and a run with ``writes_cache=False`` only reads what another run of
    the same step stored there.  ``add_embedding``: right before this run the embedding
    output (what the stream held before the first run) is added to the stream once more -
    for models that run a stretch of layers several times and feed the input in again at
    the start of each further pass.  ``mix_input``: right before this run the stream x becomes
    W [x ; x0] with x0 the embedding output and W the model's :attr:`ModelSpec.input_mix` tensor -
    the other way of feeding the input in again, a learned one.  ``more_caches``: further cache
    entries of a mixer that keeps more than one thing (a pair of mixers side by side: pages for
    one, a fixed-size state for the other), in the order of its ``extra_cache_specs()``.
    """
    layer: int
    cache: Optional[int] = None
    writes_cache: bool = True
    add_embedding: bool = False
    mix_input: bool = False
    more_caches: Tuple[int, ...] = ()


@dataclasses.dataclass(frozen=True)
class PairTableSpec:
    """A second embedding table, indexed by a hash of a token and the one before it in its sequence:
    row (previous * mul_prev + current * mul_cur) mod buckets is added to the token's embedding, and row
    ``buckets`` (the table's last) for a sequence's first token.  The previous token of every live
    sequence is kept in the cache entry ``cache`` (one 32-bit integer per slot)."""
    table: TensorSpec            # [buckets + 1, hidden]
    buckets: int
    mul_prev: int
    mul_cur: int
    cache: int


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: TensorSpec
    layers: List[LayerSpec]
    schedule: List[RunSpec]
    final_norm: PartSpec
    lm_head: TensorSpec            # optional_alias set when tied to the embedding
    #: what goes into the residual stream for token t: embedding[id] * embedding_multiplier, plus
    #: position_table[position] if the model has learned absolute positions ([max_positions, hidden])
    embedding_multiplier: float = 1.0
    position_table: Optional[TensorSpec] = None
    #: logits = logit_multiplier * (final norm . lm_head^T)
    logit_multiplier: float = 1.0
    #: tensor names a checkpoint may hold although the model does not read them
    ignorable: Tuple[str, ...] = ()
    #: a hashed table of token pairs added to the embedding (None: the model has none)
    pair_table: Optional[PairTableSpec] = None
    #: [hidden, 2 hidden]: what runs with ``mix_input`` multiply [x ; x0] by
    input_mix: Optional[TensorSpec] = None

    def num_cache_entries(self) -> int:
        used = [r.cache for r in self.schedule if r.cache is not None]
        used += [c for r in self.schedule for c in r.more_caches]
        if self.pair_table is not None:
            used.append(self.pair_table.cache)
        return (max(used) + 1) if used else 0

    def check(self) -> None:
        if not self.schedule:
            raise ValueError("a model needs at least one scheduled layer")
        if self.position_table is not None and tuple(self.position_table.shape) != (self.max_positions,
                                                                                     self.hidden_size):
            raise ValueError(f"the position table must be [{self.max_positions}, {self.hidden_size}], "
                             f"not {tuple(self.position_table.shape)}")
        if self.input_mix is not None and tuple(self.input_mix.shape) != (self.hidden_size, 2 * self.hidden_size):
            raise ValueError(f"input_mix must be [{self.hidden_size}, {2 * self.hidden_size}], "
                             f"not {tuple(self.input_mix.shape)}")
        if self.pair_table is not None and tuple(self.pair_table.table.shape) != (self.pair_table.buckets + 1,
                                                                                   self.hidden_size):
            raise ValueError("the pair table must be [buckets + 1, hidden]")
        written = set() if self.pair_table is None else {self.pair_table.cache}
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {run.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if run.add_embedding and i == 0:
                raise ValueError("schedule[0] cannot add the embedding output again: the stream "
                                 "holds nothing else yet")
            if run.mix_input and self.input_mix is None:
                raise ValueError(f"schedule[{i}] mixes the input in, but the model names no input_mix tensor")
            if run.mix_input and run.add_embedding:
                raise ValueError(f"schedule[{i}] feeds the input in again in two ways at once")
            for c in run.more_caches:
                if c < 0 or c in written or c == run.cache:
                    raise ValueError(f"schedule[{i}] names the further cache entry {c}, which is negative or taken")
                written.add(c)
            if run.cache is not None:
                if run.cache < 0:
                    raise ValueError(f"schedule[{i}] names a negative cache entry")
                if run.writes_cache:
                    if run.cache in written:
                        raise ValueError(f"schedule[{i}] writes cache entry {run.cache} "
                                         "that an earlier run already writes")
                    written.add(run.cache)
                elif run.cache not in written:
                    raise ValueError(f"schedule[{i}] reads cache entry {run.cache} "
                                     "before any run wrote it")


@dataclasses.dataclass(frozen=True)
class CacheSpec:
    """What one cache entry of a mixer needs per sequence.

    ``kind="kv"``: keys and values of ``heads`` x ``head_dim`` per token, all of them
    or only the last ``window`` tokens; ``planes=1``: one row per token and head instead of a key
    and a value row (a mixer whose keys and values are read from the same cached vector).
    ``kind="state"``: one tensor of fixed
    ``shape`` per sequence (32-bit unless ``state_dtype`` says otherwise), zeroed when
    a sequence takes the slot.  Entries with equal specs form one group with storage
    of its own.
    """
    kind: str
    heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"
    planes: int = 2

    def group_key(self):
        return (self.kind, self.heads, self.head_dim, self.window, self.shape, self.state_dtype, self.planes)
