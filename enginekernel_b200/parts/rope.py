"""Rotary position encoding with NeoX pairing (dimension j rotates with j + rot/2).

Angles: position * theta^(-2j/rot) for j < rot/2, computed in 32-bit on the host with the
reference's formula (engine/ek_model.py:164-174) and kept as 32-bit cos/sin tables of
rot/2 columns (the reference stores the doubled table in the model dtype).  Parameters:
``head_dim``, ``theta``, ``rotary_dim`` (<= head_dim; the dimensions past it are left
unrotated).  The rotation itself happens inside the mixer's kernel, which reads the
tables per token position.
"""

from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import PositionEncoding

_TABLES: Dict[tuple, tuple] = {}


@register_part("position", "rope_neox")
class RopeNeox(PositionEncoding):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.head_dim = int(self.param("head_dim"))
        self.theta = float(self.param("theta"))
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim")
        self.cos = self.sin = None
        self.num_positions = 0

    def prepare(self, max_positions: int) -> None:
        key = (str(self.device), self.theta, self.rotary_dim, max_positions)
        if key not in _TABLES:
            rot = self.rotary_dim
            inv = 1.0 / (self.theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
            t = torch.arange(max_positions, dtype=torch.float32)
            freqs = torch.outer(t, inv)
            if len(_TABLES) > 8:
                _TABLES.clear()
            _TABLES[key] = (freqs.cos().to(self.device).contiguous(),
                            freqs.sin().to(self.device).contiguous())
        self.cos, self.sin = _TABLES[key]
        self.num_positions = max_positions


@register_part("position", "rope_stretched")
class RopeStretched(PositionEncoding):
    """NeoX-paired rotation whose slow dimensions turn ``factor`` times slower (YaRN).

    With f_i = theta^(-2i/rot) for i < rot/2: let dim(t) = rot ln(original / (2 pi t)) / (2 ln theta),
    lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), rot - 1) and ramp_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1).  Dimension i turns by position * (f_i / factor * ramp_i + f_i (1 - ramp_i)),
    and cosines and sines are multiplied by 0.1 ln(factor) + 1.  Parameters: ``rotary_dim`` (rot),
    ``theta``, and ``factor``, ``original``, ``fast``, ``slow`` (without ``factor``: the plain rotation).
    With ``divide`` every frequency is divided by that number afterwards (positions interpolated
    linearly; it works without ``factor`` too).
    The tables are worked out in 64-bit on the host and kept in 32-bit, with the factor on cos and sin
    folded in, so the kernels that read ``cos`` / ``sin`` need to know nothing of it.
    """

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.rotary_dim = int(self.param("rotary_dim"))
        self.theta = float(self.param("theta"))
        self.factor = spec.params.get("factor")
        self.divide = float(spec.params.get("divide") or 1.0)
        if not self.divide > 0:
            raise ValueError("rope_stretched: divide must be positive")
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even")
        if self.factor is not None:
            self.factor = float(self.factor)
            self.original = float(self.param("original"))
            self.fast, self.slow = float(self.param("fast")), float(self.param("slow"))
            if not (self.factor > 0 and self.original > 0 and self.fast > 0 and self.slow > 0):
                raise ValueError("rope_stretched: factor, original, fast and slow must be positive")
        self.cos = self.sin = None
        self.num_positions = 0

    def frequencies(self):
        """(frequencies [rot/2] in 64-bit, factor on cos and sin)."""
        import math
        rot, half = self.rotary_dim, self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        f = self.theta ** (-2.0 * i / max(rot, 1))
        f = f / self.divide
        if self.factor is None:
            return f, 1.0

        def dim_of(turns):
            return rot * math.log(self.original / (2 * math.pi * turns)) / (2 * math.log(self.theta))

        lo = max(math.floor(dim_of(self.fast)), 0)
        hi = min(math.ceil(dim_of(self.slow)), rot - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / self.factor * ramp + f * (1.0 - ramp), 0.1 * math.log(self.factor) + 1.0

    def prepare(self, max_positions: int) -> None:
        key = ("stretched", str(self.device), self.theta, self.rotary_dim, max_positions, self.factor, self.divide,
               getattr(self, "original", None), getattr(self, "fast", None), getattr(self, "slow", None))
        if key not in _TABLES:
            f, mult = self.frequencies()
            ang = torch.outer(torch.arange(max_positions, dtype=torch.float64), f)
            if len(_TABLES) > 8:
                _TABLES.clear()
            _TABLES[key] = ((ang.cos() * mult).to(torch.float32).to(self.device).contiguous(),
                            (ang.sin() * mult).to(torch.float32).to(self.device).contiguous())
        self.cos, self.sin = _TABLES[key]
        self.num_positions = max_positions
