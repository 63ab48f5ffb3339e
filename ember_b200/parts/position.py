"""Position encodings.

Rotary, rotate-half layout (src/backend/cpu/cpu_backend.cpp:85-88, 263-272):
inv_freq_i = 1 / powf(float(theta), float(2i) / float(rotary_dim)) computed in fp32; the angle
float(pos) * inv_freq_i and its sine and cosine are fp32; pairs are (x_i, x_{i + rotary_dim/2}).
The rotation itself runs inside the mixer's fused norm + rotation + cache-write kernel; this
part owns the frequency table, so an encoding with other frequencies (or none) is another
part with the same interface.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..config.spec import ConfigError
from .base import PositionEncoding, Runtime
from .registry import register_part


class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim:
            raise ConfigError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        if getattr(spec, "scaling_factor", 0.0) and not (spec.scaling_factor > 0 and spec.scaling_original > 0 and spec.scaling_fast > 0
                                                         and spec.scaling_slow > 0 and spec.theta > 1):
            raise ConfigError("rotary scaling needs a positive factor, original length, fast and slow turns, and a base above 1")
        self._table = None

    def _scaled(self, f: np.ndarray) -> np.ndarray:
        """Frequencies stretched for long contexts: a ramp over the pair index from the pairs that turn more than
        ``fast`` times over the original length (kept) to those that turn fewer than ``slow`` times (divided by the
        factor)."""
        s = self.spec
        dims = s.rotary_dim

        def pair_at(turns: float) -> float:
            return dims * math.log(s.scaling_original / (2.0 * math.pi * turns)) / (2.0 * math.log(s.theta))

        lo = max(math.floor(pair_at(s.scaling_fast)), 0)
        hi = min(math.ceil(pair_at(s.scaling_slow)), dims - 1)
        ramp = np.clip((np.arange(dims // 2, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / s.scaling_factor * ramp + f * (1.0 - ramp)

    def magnitude(self) -> float:
        """What cosines and sines are multiplied by: 0.1 ln(factor) + 1 under scaling, else 1."""
        factor = getattr(self.spec, "scaling_factor", 0.0)
        return 0.1 * math.log(factor) + 1.0 if factor else 1.0

    def inv_freq(self) -> np.ndarray:
        r = self.spec.rotary_dim
        linear = float(getattr(self.spec, "linear_factor", 1.0))
        if linear != 1.0:                               # every frequency divided by the factor, in float64, rounded once
            if not linear > 0 or getattr(self.spec, "scaling_factor", 0.0):
                raise ConfigError("linear rotary scaling needs a positive factor and excludes the stretched frequencies")
            return (np.power(float(self.spec.theta), -2.0 * np.arange(r // 2, dtype=np.float64) / r) / linear).astype(np.float32)
        if getattr(self.spec, "scaling_factor", 0.0):
            f = np.power(float(self.spec.theta), -2.0 * np.arange(r // 2, dtype=np.float64) / r)
            return self._scaled(f).astype(np.float32)
        if getattr(self.spec, "frequency_precision", "float32") == "float64":
            return np.power(float(self.spec.theta), -2.0 * np.arange(r // 2, dtype=np.float64) / r).astype(np.float32)
        i = np.arange(r // 2, dtype=np.float32)
        exponent = (np.float32(2.0) * i) / np.float32(r)                      # float(2i) / float(D)
        return (np.float32(1.0) / np.power(np.float32(self.spec.theta), exponent, dtype=np.float32)).astype(np.float32)

    def rotary_table(self, rt: Runtime):
        if self._table is None or self._table.device != rt.device:
            self._table = torch.from_numpy(self.inv_freq()).to(rt.device)
        return self._table, self.spec.rotary_dim

    def table_key(self):
        s = self.spec
        return (s.rotary_dim, float(s.theta), getattr(s, "frequency_precision", "float32"), getattr(s, "layout", "half"),
                getattr(s, "scaling_factor", 0.0), getattr(s, "scaling_original", 0.0), getattr(s, "scaling_fast", 0.0),
                getattr(s, "scaling_slow", 0.0), getattr(s, "linear_factor", 1.0))


class NoPosition(PositionEncoding):
    graph_safe = True


register_part("position", "rope", RotaryEmbedding)
register_part("position", "none", NoPosition)
