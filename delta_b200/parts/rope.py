"""Rotary position encoding.

Pair j of a head is rotated by the angle  position / (scale * theta^(2j/head_dim))
(reference: DELTA/Engine/DELTA/model.py:165-175, ``apply_rope`` with
``rope_scale`` and ``rope_theta``).  The reference pairs neighbouring elements
(2j, 2j+1) because it runs checkpoints whose q and k rows were permuted by a
converter; on the rows of an unconverted model folder the same function pairs
(j, j + head_dim/2), which is the default here.  ``interleaved=True`` gives the
reference's pairing.

``scaling`` {factor, low, high, original} stretches long wavelengths (the Llama 3.1 rule): with wavelength
l = 2 pi / f, a frequency f is kept where l < original / high, divided by ``factor`` where l > original / low, and
between the two blended, (1 - s) f / factor + s f with s = (original / l - low) / (high - low).

``scaling`` {factor, original, fast, slow} is the other rule ("YaRN"): with pair(t) = head_dim ln(original / (2 pi t)) / (2 ln theta)
the (fractional) pair whose wave makes t turns over the original length, lo = max(floor(pair(fast)), 0),
hi = min(ceil(pair(slow)), head_dim - 1) and ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1), pair j turns by
f_j / factor * ramp_j + f_j (1 - ramp_j), and cos and sin are both multiplied by 0.1 ln(factor) + 1.

Cos and sin are tabulated once per (head_dim, theta, scale) in 64 bit and
rounded to 32 bit, so the kernels do no trigonometry and the angles carry no
32-bit rounding of a large position times a small frequency.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import POSITION_ENCODINGS, PositionEncoding

_TABLES: dict = {}


@POSITION_ENCODINGS.register("rotary")
class RotaryPositions(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int, interleaved: bool = False, scale: float = 1.0,
                 scaling: Optional[dict] = None):
        if head_dim % 2:
            raise ValueError(f"rotary positions need an even head size, got {head_dim}")
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self.interleaved = bool(interleaved)
        self.scale = float(scale)
        self.scaling = self.ramp = None
        if scaling and ("fast" in scaling or "slow" in scaling):
            self.ramp = tuple(float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
            if min(self.ramp) <= 0 or self.theta <= 1.0:
                raise ValueError("rotary scaling: factor, original, fast and slow must be positive and the base above 1")
        elif scaling:
            self.scaling = tuple(float(scaling[k]) for k in ("factor", "low", "high", "original"))
            if self.scaling[2] == self.scaling[1]:
                raise ValueError("rotary scaling: 'high' and 'low' must differ")

    def frequencies(self) -> torch.Tensor:
        """[head_dim/2] float64: the angle a position advances every pair by."""
        half = self.head_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        inv = 1.0 / (self.scale * self.theta ** (2.0 * j / self.head_dim))
        if self.scaling is not None:
            factor, low, high, original = self.scaling
            wave = 2.0 * math.pi / inv
            s = (original / wave - low) / (high - low)
            blend = (1.0 - s) * inv / factor + s * inv
            inv = torch.where(wave < original / high, inv, torch.where(wave > original / low, inv / factor, blend))
        if self.ramp is not None:
            factor, original, fast, slow = self.ramp

            def pair(turns):
                return self.head_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(pair(fast)), 0)
            hi = min(math.ceil(pair(slow)), self.head_dim - 1)
            ramp = ((j - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            inv = inv / factor * ramp + inv * (1.0 - ramp)
        return inv

    def magnitude(self) -> float:
        """The factor on cos and sin (1 unless the scaling rule has one)."""
        return 0.1 * math.log(self.ramp[0]) + 1.0 if self.ramp is not None else 1.0

    def table_cpu(self) -> torch.Tensor:
        """[max_positions, head_dim/2, 2] float32: cos and sin of every angle."""
        inv = self.frequencies()
        ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        return (torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1) * self.magnitude()).to(torch.float32).contiguous()

    def table(self, device) -> torch.Tensor:
        key = (self.head_dim, self.theta, self.scale, self.scaling, self.ramp, self.max_positions, str(device))
        if key not in _TABLES:
            _TABLES[key] = self.table_cpu().to(device)
        return _TABLES[key]
