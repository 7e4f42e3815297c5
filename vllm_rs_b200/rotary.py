"""Rotary-embedding frequency tables built on the host (double precision)."""
from __future__ import annotations

import math

import numpy as np


def rotary_frequencies(dims: int, base: float, scaling: dict | None = None) -> tuple[np.ndarray, float]:
    """Per-pair angular frequencies f[i] (i < dims / 2; the angle of pair i at position p is p * f[i]) and the
    factor that multiplies cos and sin.

    Without `scaling`: f[i] = base^(-2 i / dims), factor 1.  With YaRN scaling {factor s, original L, fast, slow}:
    pairs that turn more than `fast` times over the original length L keep their frequency, pairs that turn fewer
    than `slow` times are slowed by s, and a linear ramp blends in between.  The pair index at which a frequency
    makes t turns over L is  d(t) = dims * ln(L / (2 pi t)) / (2 ln base);  lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), dims - 1), r[i] = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    f'[i] = f[i] / s * r[i] + f[i] * (1 - r[i]), factor = 0.1 ln(s) + 1."""
    half = dims // 2
    idx = np.arange(half, dtype=np.float64)
    freq = np.power(float(base), -2.0 * idx / dims)
    if not scaling:
        return freq, 1.0
    s, length = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns: float) -> float:
        return dims * math.log(length / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((idx - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / s * ramp + freq * (1.0 - ramp), 0.1 * math.log(s) + 1.0


def banded_rotary_frequencies(dims: int, base: float, scaling: dict | None = None) -> np.ndarray:
    """Per-pair angular frequencies with scaling by wavelength band {factor s, low, high, original L}: with the
    wavelength lam = 2 pi / f of a pair, short ones (lam < L / high) keep f, long ones (lam > L / low) get f / s, and
    in between  f' = (1 - t) f / s + t f  with  t = (L / lam - low) / (high - low).  No magnitude factor."""
    idx = np.arange(dims // 2, dtype=np.float64)
    freq = np.power(float(base), -2.0 * idx / dims)
    if not scaling:
        return freq
    s, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
    length = float(scaling["original"])
    lam = 2.0 * math.pi / freq
    t = (length / lam - low) / (high - low)
    mid = (1.0 - t) * freq / s + t * freq
    return np.where(lam < length / high, freq, np.where(lam > length / low, freq / s, mid))
