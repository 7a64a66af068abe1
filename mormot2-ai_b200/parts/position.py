"""Position encodings. A mixer asks its encoding for the inverse frequencies and for how many
values of a head rotate; the angle of a position is formed in the kernel as the float32
product inv_freq[i] · pos.

``rope_half`` is the rotary encoding in the rotate-half pairing (i, i + rot_dim/2) with
inv_freq[i] = 1 / f32(theta ^ f32(2i / rot_dim)), each step rounded to float32 as the
reference does (``decoder.pas:1733-1736``; angles ``:2539-2561``); with ``rounding`` = "once"
the frequencies theta^(−2i / rot_dim) are formed in float64 and rounded to float32 once.
``none`` rotates nothing.

``rope_pairs`` has the same frequencies and angles but turns neighbours: value 2i with value
2i + 1. A mixer whose rotated values only ever meet in a dot product of two vectors turned the
same way (queries and keys) may serve it with the rotate-half kernels by reordering the rows
of the projections that produce those values once at load: ``half_order()`` gives the order
(old index of every new place) that makes pair i land on the places i and i + rot_dim/2.

``rope_yarn`` is the same rotation with YaRN's frequencies: with
d(t) = dims · ln(original / (2π t)) / (2 ln theta), lo = max(floor(d(fast)), 0),
hi = min(ceil(d(slow)), dims − 1) and ramp_i = clamp((i − lo) / max(hi − lo, 0.001), 0, 1),
frequency i is f_i · ((1 − ramp_i) + ramp_i / factor): fast-turning pairs keep their
frequency, slow ones are stretched by ``factor``. Cosine and sine are both multiplied by
``amplitude`` = 0.1 · ln(factor) + 1. An encoding's ``amplitude`` is 1 unless it says
otherwise; a mixer passes it to the kernel that rotates.

``rope_scaled_bands`` is the same rotation with the frequencies scaled by wavelength, as
Llama 3.1 scales them: with the wavelength l = 2π / f, frequencies with l < original / high
stay, those with l > original / low become f / factor, and between the two, with
s = (original / l − low) / (high − low), f' = (1 − s) · f / factor + s · f.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

from ..errors import ConfigError
from .base import POSITIONS, Part


def rope_inverse_frequencies(theta: float, rot_dim: int) -> np.ndarray:
    out = np.empty(rot_dim // 2, dtype=np.float32)
    for i in range(rot_dim // 2):
        exponent = np.float32((2 * i) / rot_dim)
        power = np.float32(math.exp(math.log(theta) * float(exponent)))
        out[i] = np.float32(1.0 / float(power))
    return out


class RopeHalf(Part):
    capturable = True
    amplitude = 1.0

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.theta = float(spec.params["theta"])
        self.rot_dim = int(spec.params["rot_dim"])
        if self.rot_dim <= 0 or self.rot_dim % 2:
            raise ConfigError(f"a rotary encoding over {self.rot_dim} values of a head")
        self.rounding = spec.params.get("rounding", "stepwise")
        if self.rounding not in ("stepwise", "once"):
            raise ConfigError(f"rounding \"{self.rounding}\" of the frequencies (stepwise, once)")
        self.inv_freq: Optional[torch.Tensor] = None

    def bind(self, weights, rt) -> None:
        if self.rounding == "once":
            i = np.arange(self.rot_dim // 2, dtype=np.float64)
            f = np.exp(-np.log(self.theta) * 2.0 * i / self.rot_dim).astype(np.float32)
        else:
            f = rope_inverse_frequencies(self.theta, self.rot_dim)
        self.inv_freq = torch.from_numpy(f).to(rt.device)

    def frequencies(self) -> Tuple[Optional[torch.Tensor], int]:
        return self.inv_freq, self.rot_dim


class RopePairs(RopeHalf):
    pairing = "neighbours"

    def half_order(self, size: int) -> list:
        """For a vector of ``size`` values whose first ``rot_dim`` turn as neighbours: the
        order [0, 2, 4, ..., 1, 3, 5, ..., rest] in which the rotate-half pairing turns the
        same pairs by the same angles."""
        r = self.rot_dim
        if size < r:
            raise ConfigError(f"{r} rotating values of a vector of {size}")
        return list(range(0, r, 2)) + list(range(1, r, 2)) + list(range(r, size))


def yarn_inverse_frequencies(theta: float, rot_dim: int, factor: float, original: float,
                             fast: float, slow: float) -> np.ndarray:
    """Float64 arithmetic, rounded to float32 once at the end."""
    half = rot_dim // 2
    i = np.arange(half, dtype=np.float64)
    f = np.exp(-np.log(theta) * 2.0 * i / rot_dim)

    def dim_of(turns: float) -> float:
        return rot_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), rot_dim - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).astype(np.float32)


class RopeYarn(RopeHalf):
    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.factor, self.original = float(p["factor"]), float(p["original"])
        self.fast, self.slow = float(p["fast"]), float(p["slow"])
        if min(self.factor, self.original, self.fast, self.slow) <= 0:
            raise ConfigError("YaRN scaling: factor, original, fast and slow are positive")
        self.amplitude = 0.1 * math.log(self.factor) + 1.0

    def bind(self, weights, rt) -> None:
        self.inv_freq = torch.from_numpy(yarn_inverse_frequencies(
            self.theta, self.rot_dim, self.factor, self.original, self.fast,
            self.slow)).to(rt.device)


def banded_inverse_frequencies(theta: float, rot_dim: int, factor: float, low: float,
                               high: float, original: float) -> np.ndarray:
    """Float64 arithmetic, rounded to float32 once at the end."""
    half = rot_dim // 2
    f = np.exp(-np.log(theta) * 2.0 * np.arange(half, dtype=np.float64) / rot_dim)
    wavelength = 2.0 * math.pi / f
    s = (original / wavelength - low) / (high - low) if high != low else np.ones(half)
    blended = (1.0 - s) * f / factor + s * f
    out = np.where(wavelength < original / high, f,
                   np.where(wavelength > original / low, f / factor, blended))
    return out.astype(np.float32)


class RopeScaledBands(RopeHalf):
    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.factor, self.original = float(p["factor"]), float(p["original"])
        self.low, self.high = float(p["low"]), float(p["high"])
        if min(self.factor, self.original, self.low, self.high) <= 0:
            raise ConfigError("frequency scaling: factor, original, low and high are positive")

    def bind(self, weights, rt) -> None:
        self.inv_freq = torch.from_numpy(banded_inverse_frequencies(
            self.theta, self.rot_dim, self.factor, self.low, self.high,
            self.original)).to(rt.device)


class NoPosition(Part):
    capturable = True
    amplitude = 1.0

    def frequencies(self) -> Tuple[Optional[torch.Tensor], int]:
        return None, 0


POSITIONS.register("rope_half", RopeHalf)
POSITIONS.register("rope_pairs", RopePairs)
POSITIONS.register("rope_yarn", RopeYarn)
POSITIONS.register("rope_scaled_bands", RopeScaledBands)
POSITIONS.register("none", NoPosition)
