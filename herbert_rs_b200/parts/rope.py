"""Rotary position encoding: the cos/sin tables a mixer rotates with.

Reference (crates/backends/backend_common/src/loader_common.rs:179-202), all in float32:
  inv_freq_i = 1 / theta^(2i / rot)   for i < rot/2
  angle(pos, i) = float(pos) * inv_freq_i;  tables cos, sin of shape [max_position, rot/2].
The rotation itself pairs element j with j + rot/2 (kernels.rs:739-759) and is fused into the
mixer's cache-write kernel.
"""

from __future__ import annotations

import torch

from ..errors import ConfigError
from ..registry import register_part
from .base import Part


def rope_tables(rotary_dim: int, theta: float, max_position: int):
    """float32 tables on the CPU; every intermediate is float32, as in the reference."""
    half = rotary_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    exponent = (2.0 * i) / torch.tensor(float(rotary_dim), dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    pos = torch.arange(max_position, dtype=torch.float32)
    ang = pos[:, None] * inv_freq[None, :]
    return torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


_TABLES: dict = {}


class RotaryEncoding(Part):
    """Holds the tables on the device; equal specs on one device share them."""

    def __init__(self, spec, rt):
        self.rotary_dim = spec.rotary_dim
        self.max_position = spec.max_position
        key = (spec.rotary_dim, float(spec.theta), spec.max_position, str(rt.device))
        if key not in _TABLES:
            cos, sin = rope_tables(spec.rotary_dim, spec.theta, spec.max_position)
            _TABLES[key] = (cos.to(rt.device), sin.to(rt.device))
        self.cos, self.sin = _TABLES[key]


def scaled_frequencies(spec):
    """(f [rotary_dim/2] float64, m) of a `ScaledRotarySpec` (its docstring has the formulas)."""
    import math
    half = spec.rotary_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / spec.rotary_dim)
    if spec.factor is None:
        return f, 1.0

    def d(t):
        return spec.rotary_dim * math.log(spec.original / (2.0 * math.pi * t)) / (2.0 * math.log(spec.theta))
    lo = max(math.floor(d(spec.fast)), 0)
    hi = min(math.ceil(d(spec.slow)), spec.rotary_dim - 1)
    r = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / spec.factor * r + f * (1.0 - r), 0.1 * math.log(spec.factor) + 1.0


class ScaledRotary(Part):
    """Frequencies on the device (float32) and the constant that multiplies cos and sin; the kernels
    take the angle position * frequency in float, so no table bounds the position."""

    def __init__(self, spec, rt):
        self.rotary_dim = spec.rotary_dim
        f, self.mscale = scaled_frequencies(spec)
        self.freq = f.to(torch.float32).to(rt.device)


register_part("position", "rope", RotaryEncoding)
register_part("position", "scaled_rope", ScaledRotary)


def pair_frequencies(rotary_dim: int, theta: float, linear_factor: float = 1.0, band_scaling=None) -> torch.Tensor:
    """theta^(-2m / rotary_dim) / linear_factor for m < rotary_dim / 2, computed in float64, as float32.
    `band_scaling` (factor, low, high, original): a frequency whose wavelength l = 2 pi / f is shorter than
    original / high stays, one longer than original / low is divided by factor, and between the two it is
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    m = torch.arange(rotary_dim // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * m / rotary_dim) / float(linear_factor)
    if band_scaling is not None:
        import math
        factor, low, high, original = (float(v) for v in band_scaling)
        if not (factor > 0.0 and original > 0.0 and high > low >= 0.0):
            raise ConfigError(f"band scaling of rotary frequencies needs factor > 0, original > 0 and high > low >= 0, got {band_scaling}")
        wavelength = 2.0 * math.pi / f
        s = (original / wavelength - low) / (high - low)
        mixed = (1.0 - s) * f / factor + s * f
        long_ = wavelength > original / low if low > 0.0 else torch.zeros_like(f, dtype=torch.bool)
        f = torch.where(wavelength < original / high, f, torch.where(long_, f / factor, mixed))
    return f.to(torch.float32)


class RotaryPairs(Part):
    """Frequencies of a `RotaryPairsSpec` on the device; the kernels take the angle position * frequency in
    float and the accurate sine and cosine, so no table bounds the position."""

    def __init__(self, spec, rt):
        if spec.rotary_dim % 2 or spec.rotary_dim < 0:
            raise ConfigError(f"{spec.rotary_dim} rotated channels have no pairs")
        if spec.layout not in ("interleaved", "halves"):
            raise ConfigError(f"unknown layout of rotated pairs {spec.layout!r}: interleaved, halves")
        self.rotary_dim = spec.rotary_dim
        self.halves = spec.layout == "halves"
        self.freq = pair_frequencies(spec.rotary_dim, spec.theta, spec.linear_factor,
                                     getattr(spec, "band_scaling", None)).to(rt.device) if spec.rotary_dim else None


register_part("position", "rope_pairs", RotaryPairs)
