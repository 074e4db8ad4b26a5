"""Rotary position encoding with half-split pairing.

inv_freq_i = theta^(-2i/rotary_dim); angle = position * inv_freq_i;
out[i] = x[i]*cos - x[i+r/2]*sin; out[i+r/2] = x[i]*sin + x[i+r/2]*cos
(`model.py:131-145`; the engine builds the tables in f64 and stores f32,
`engine/src/ops.rs:101-115`; kernel `engine/kernels/kernels.cu:1677-1706`).
The tables are fp32 in both engine dtypes and the rotation is fp32 arithmetic.
"""
from __future__ import annotations

import torch

from ..config.model_config import PositionSpec
from .base import POSITIONS, PositionEncoding


_TABLES = {}     # (theta, rotary_dim, positions, device) -> (cos, sin), read-only


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PositionSpec):
        if spec.rotary_dim % 2 != 0 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be a positive even number, got {spec.rotary_dim}")
        self.spec = spec
        self.cos = None
        self.sin = None

    def bind(self, tensors, dtype, device):
        # layers with the same rotation share one pair of tables (a model of 32 layers
        # with 131,072 positions would otherwise hold 32 identical pairs of 33 MB)
        key = (float(self.spec.theta), self.spec.rotary_dim, self.spec.max_positions,
               str(torch.device(device)))
        hit = _TABLES.get(key)
        if hit is None:
            half = self.spec.rotary_dim // 2
            i = torch.arange(half, dtype=torch.float64)
            inv_freq = torch.pow(torch.tensor(self.spec.theta, dtype=torch.float64),
                                 -2.0 * i / self.spec.rotary_dim)
            pos = torch.arange(self.spec.max_positions, dtype=torch.float64)
            ang = torch.outer(pos, inv_freq)
            hit = (ang.cos().to(torch.float32).contiguous().to(device),
                   ang.sin().to(torch.float32).contiguous().to(device))
            if len(_TABLES) >= 8:
                _TABLES.pop(next(iter(_TABLES)))
            _TABLES[key] = hit
        self.cos, self.sin = hit

    def rotation(self):
        return self.cos, self.sin, self.spec.rotary_dim


POSITIONS.register("rope", RotaryEncoding)


class InterleavedRotary(PositionEncoding):
    """Rotation of neighbouring pairs: features (2i, 2i+1), i < rotary_dim / 2, of a head
    turn by the angle position * theta^(-2i / rotary_dim); features from rotary_dim on
    pass unchanged.  (u, v) -> (u cos a - v sin a, v cos a + u sin a).  The frequencies
    are float32 numbers and the angle is a float32 product taken in the kernel, so there
    is no table over positions and no longest position."""

    split_halves = False       # which features pair: neighbours (2i, 2i + 1)

    def __init__(self, spec: PositionSpec):
        if spec.rotary_dim % 2 != 0 or spec.rotary_dim < 0:
            raise ValueError(f"rotary_dim must be even and not negative, got {spec.rotary_dim}")
        self.spec = spec
        self.freq = None

    def bind(self, tensors, dtype, device):
        n = self.spec.rotary_dim
        i = torch.arange(n // 2, dtype=torch.float64)
        # taken in float64 and rounded once, so every frequency is the nearest float32
        self.freq = (float(self.spec.theta) ** (-2.0 * i / n)).to(torch.float32).to(device) if n else None

    def frequencies(self):
        return self.freq, self.spec.rotary_dim


POSITIONS.register("rope_interleaved", InterleavedRotary)


class YarnRotary(PositionEncoding):
    """Half-split pairs (feature i with i + rotary_dim / 2) whose frequencies are stretched for
    contexts beyond the one the model was trained at.  With f_i = theta^(-2i / n):
        dim(t) = n ln(original / (2 pi t)) / (2 ln theta),
        lo = max(floor(dim(fast)), 0),  hi = min(ceil(dim(slow)), n - 1),
        ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
        frequency_i = f_i / factor * ramp_i + f_i * (1 - ramp_i),
    and cos and sin are multiplied by 0.1 ln(factor) + 1 (`magnitude()`).  Without the options
    `factor`, `original`, `fast`, `slow` (the spec's `extra`) the frequencies are the base's and the
    magnitude is 1.  The angle is a float32 product of position and frequency taken in the kernel."""

    split_halves = True        # which features pair: i with i + rotary_dim / 2

    def __init__(self, spec: PositionSpec, scaling=None):
        if spec.rotary_dim % 2 != 0 or spec.rotary_dim < 0:
            raise ValueError(f"rotary_dim must be even and not negative, got {spec.rotary_dim}")
        self.spec = spec
        self.scaling = dict(scaling) if scaling else None
        self.freq = None

    def _frequencies(self) -> torch.Tensor:
        import math
        n, base = self.spec.rotary_dim, float(self.spec.theta)
        i = torch.arange(n // 2, dtype=torch.float64)
        f = base ** (-2.0 * i / n)
        sc = self.scaling
        if sc:
            def dim_of(turns):
                return n * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
            lo = max(math.floor(dim_of(sc["fast"])), 0)
            hi = min(math.ceil(dim_of(sc["slow"])), n - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        return f.to(torch.float32)

    def magnitude(self) -> float:
        import math
        return 0.1 * math.log(self.scaling["factor"]) + 1.0 if self.scaling else 1.0

    def bind(self, tensors, dtype, device):
        self.freq = self._frequencies().to(device) if self.spec.rotary_dim else None

    def frequencies(self):
        return self.freq, self.spec.rotary_dim


POSITIONS.register("rope_yarn", lambda spec: YarnRotary(spec, spec.scaling))
# split halves with the base's own frequencies and the angle taken in the kernel as an fp32
# product (no table over positions, no longest position)
POSITIONS.register("rope_halves", lambda spec: YarnRotary(spec, None))
