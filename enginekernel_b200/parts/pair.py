"""Two mixers side by side: both read the same normalised input, and the layer's result is
weight_a * first(h) + weight_b * second(h).

Each of the two is a registered mixer of its own (any kinds), built from its own PartSpec with its own tensors and its
own cache entry: the first one's is the run's ``cache``, the second one's the run's first entry of ``more_caches``.
The sum is not formed here: the part hands both results and the two weights on as a
:class:`~enginekernel_b200.parts.base.WeightedPair`, and the kernel that reads the result next (a block's norm)
forms it on its way through the row (the ``sandwich`` block takes pairs).
Each side works in scratch buffers of its own, so that the first result outlives the second mixer's run.

Parameters: ``first``, ``second`` (PartSpecs of role mixer), ``weight_first``, ``weight_second``.
"""

from __future__ import annotations

import dataclasses

from ..registry import lookup_part, register_part
from .base import Mixer, WeightedPair


class _SideWorkspace:
    """A workspace whose buffers carry a side's name, over the step's workspace."""

    def __init__(self, inner, prefix):
        self.inner, self.prefix, self.device = inner, prefix, inner.device

    def get(self, name, shape, dtype):
        return self.inner.get(self.prefix + name, shape, dtype)

    def bytes(self):
        return self.inner.bytes()


@register_part("mixer", "mixer_pair")
class MixerPair(Mixer):
    @classmethod
    def _sides(cls, spec):
        return [spec.params["first"], spec.params["second"]]

    @classmethod
    def tensors(cls, spec):
        out = []
        for side in cls._sides(spec):
            out += lookup_part("mixer", side.kind).tensors(side)
        return out

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.sides = [lookup_part("mixer", s.kind)(s, dtype, device) for s in self._sides(spec)]
        self.weights = (float(self.param("weight_first")), float(self.param("weight_second")))
        if any(s.cache_spec() is None for s in self.sides):
            raise ValueError("mixer_pair: both mixers must keep something per sequence")

    def cache_spec(self):
        return self.sides[0].cache_spec()

    def extra_cache_specs(self):
        return [self.sides[1].cache_spec()] + self.sides[0].extra_cache_specs() + self.sides[1].extra_cache_specs()

    def load(self, tensors):
        for s in self.sides:
            s.load(tensors)

    def prepare(self, max_positions):
        for s in self.sides:
            s.prepare(max_positions)

    def begin_step(self, ctx):
        for s in self.sides:
            s.begin_step(ctx)

    def bytes_read_per_step(self, n_tokens):
        return sum(s.bytes_read_per_step(n_tokens) for s in self.sides)

    def forward(self, x, ctx, entry, writes_cache=True):
        if not isinstance(entry, (list, tuple)) or len(entry) != 2:
            raise ValueError("mixer_pair: the run must name one cache entry for each of the two mixers")
        results = []
        for i, (side, view) in enumerate(zip(self.sides, entry)):
            sub = dataclasses.replace(ctx, workspace=_SideWorkspace(ctx.workspace, f"side{i}_"))
            results.append(side.forward(x, sub, view, writes_cache))
        return WeightedPair(results[0], self.weights[0], results[1], self.weights[1])
