"""Rotary position encoding, rotate-half layout.

Frequencies as the reference builds them, in float32
(crates/synaptix-ops/src/pos/rope_cache.rs:16-38): ``f_i = theta^(-(2 i)/d)``,
angle ``= position * f_i``.  Rotation (crates/synaptix-ops/src/pos/rope.rs:84-100):
for ``i < d/2``: ``o[i] = x[i] cos - x[i+d/2] sin``, ``o[i+d/2] = x[i] sin + x[i+d/2] cos``;
elements at and above ``rotary_dim`` pass through.

The reference tabulates cos and sin per position (and casts the tables to the
compute dtype on its graph path, model.rs:1404-1407); here the kernel computes
the angle, sine and cosine in float32 from the position, so there is no table
capacity and no rounding of the table.
"""
from __future__ import annotations

import math
from typing import NamedTuple

import numpy as np
import torch

from .base import PositionEncoding, Runtime


def rotary_inv_freq(theta: float, rotary_dim: int) -> np.ndarray:
    """``theta^(-(2i)/rotary_dim)`` for ``i < rotary_dim/2``, computed in float32."""
    i = np.arange(rotary_dim // 2, dtype=np.float32)
    exponent = -(np.float32(2.0) * i) / np.float32(rotary_dim)
    return np.power(np.float32(theta), exponent).astype(np.float32)


# one device tensor per (theta, rotary_dim, device): layers with the same rotation share it, and what a step derives
# from it (a table of cosines and sines) is made once a step, not once a layer
_INV_FREQ = {}


class RotaryHalf(PositionEncoding):
    """``scaling`` (a ``FrequencyRamp``): the slow frequencies are stretched and cos and sin both multiplied by
    ``magnitude``; the frequencies are then formed in 64-bit and rounded once.  A kernel that rotates for a part with such
    an encoding multiplies by ``magnitude`` (the parts that take one say so)."""
    pairs = False

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None, scaling: "FrequencyRamp" = None):
        self.scaling = scaling
        self.magnitude = 1.0 if scaling is None else scaling.magnitude()
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.theta = float(theta)
        self.inv_freq = None

    def bind(self, tensors, rt: Runtime) -> None:
        key = (self.theta, self.rotary_dim, self.scaling, str(rt.device))
        if key not in _INV_FREQ:
            if self.scaling is None:
                f = rotary_inv_freq(self.theta, self.rotary_dim)
            else:
                i = np.arange(self.rotary_dim // 2, dtype=np.float64)
                f = np.power(np.float64(self.theta), -2.0 * i / self.rotary_dim)
                f = self.scaling.apply(f, self.theta, self.rotary_dim).astype(np.float32)
            _INV_FREQ[key] = torch.from_numpy(f).to(rt.device)
        self.inv_freq = _INV_FREQ[key]

    def rotation(self):
        return self.inv_freq, self.rotary_dim


class RotaryPairs(RotaryHalf):
    """The same angles with NEIGHBOURING elements paired: element ``2i`` with ``2i + 1`` (the interleaved layout),
    ``(u, v) -> (u cos - v sin, v cos + u sin)`` at angle ``position * theta^(-2i / rotary_dim)``.  Kernels that
    rotate ask ``pairs``: ``True`` here, ``False`` for the rotate-half layout."""
    pairs = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None, scaling: "FrequencyRamp" = None):
        super().__init__(head_dim, theta, rotary_dim, scaling)

    def bind(self, tensors, rt: Runtime) -> None:
        # frequencies to the nearest 32-bit value (formed in 64-bit, rounded once)
        key = ("pairs", self.theta, self.rotary_dim, self.scaling, str(rt.device))
        if key not in _INV_FREQ:
            i = np.arange(self.rotary_dim // 2, dtype=np.float64)
            f = np.power(np.float64(self.theta), -2.0 * i / self.rotary_dim)
            if self.scaling is not None:
                f = self.scaling.apply(f, self.theta, self.rotary_dim)
            _INV_FREQ[key] = torch.from_numpy(f.astype(np.float32)).to(rt.device)
        self.inv_freq = _INV_FREQ[key]


class FrequencyRamp(NamedTuple):
    """Context extension by stretching the slow frequencies (the YaRN scheme): with ``dim(t) = dims ln(original /
    (2 pi t)) / (2 ln base)``, ``lo = max(floor(dim(fast)), 0)``, ``hi = min(ceil(dim(slow)), dims - 1)`` and
    ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, pair ``i`` turns at ``f_i / factor * ramp_i + f_i (1 -
    ramp_i)``, and cos and sin are both multiplied by ``0.1 ln(factor) + 1``."""
    factor: float
    original: float
    fast: float
    slow: float

    def magnitude(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0

    def apply(self, f: np.ndarray, base: float, dims: int) -> np.ndarray:
        def dim_of(t):
            return dims * math.log(self.original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(dim_of(self.fast)), 0)
        hi = min(math.ceil(dim_of(self.slow)), dims - 1)
        i = np.arange(f.shape[0], dtype=np.float64)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / self.factor * ramp + f * (1.0 - ramp)


class NoPosition(PositionEncoding):
    """Queries and keys are used as they are."""
