"""Rotary position encoding as a table of angles."""
from __future__ import annotations

import math

import torch

from ..errors import Unsupported
from .base import PositionEncoding, register_position


def inverse_frequencies(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """theta^(-2p/D) for pair p (D: the rotated part of a head), in float64 (apps/engine/src/ops.rs:128-131 of
    MythEclipse/llm), then config.json's `rope_scaling` of type llama3: pairs
    whose wavelength exceeds original/low_freq_factor are slowed by `factor`,
    those below original/high_freq_factor are kept, and the band between is
    blended linearly in original/wavelength."""
    pairs = torch.arange(head_dim // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * pairs / head_dim)
    if not scaling:
        return freq
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind == "default":
        return freq
    if kind == "ramp":
        return _ramp_scaled(freq, head_dim, theta, scaling)
    if kind == "linear":                               # positions stretched by `factor`: every frequency divided by it
        return freq / float(scaling["factor"])
    if kind != "llama3":
        raise Unsupported(f"rope scaling of type '{kind}'")
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    wavelength = 2.0 * math.pi / freq
    smooth = (original / wavelength - low) / (high - low)
    blended = (1.0 - smooth) * freq / factor + smooth * freq
    out = torch.where(wavelength > original / low, freq / factor, blended)
    return torch.where(wavelength < original / high, freq, out)


def _ramp_scaled(freq, dims: int, theta: float, scaling: dict) -> torch.Tensor:
    """Frequencies scaled by bands: with dim(t) = dims ln(original / (2 pi t)) /
    (2 ln theta) the pair index at which a wave makes t turns over the original context, pairs below
    lo = floor(dim(fast)) keep their frequency, pairs above hi = ceil(dim(slow)) are slowed by `factor`,
    and those between are blended linearly in the pair index."""
    factor, original = float(scaling["factor"]), float(scaling["original"])
    fast, slow = float(scaling["fast"]), float(scaling["slow"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), dims - 1)
    pairs = torch.arange(dims // 2, dtype=torch.float64)
    ramp = torch.clamp((pairs - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp)


def table_magnitude(scaling: dict | None) -> float:
    """What multiplies every cosine and sine of the table: 0.1 ln(factor) + 1 for the 'ramp' scaling, else 1."""
    if scaling and scaling.get("rope_type", scaling.get("type", "default")) == "ramp":
        return 0.1 * math.log(float(scaling["factor"])) + 1.0
    return 1.0


class Rope(PositionEncoding):
    """Holds a float32 table [positions, n] on the device, n = rotary_dim or head_dim: cos
    of position * inv_freq[p] in columns [0, n/2), sin in [n/2, n). Angles are computed in
    float64 and rounded once. With n < head_dim the elements of a head beyond n are not
    rotated (the rope dimension count of apps/engine/src/model.rs:93-95 of MythEclipse/llm)."""

    def __init__(self, spec):
        if spec.pairing not in ("half", "interleaved"):
            raise Unsupported(f"rope pairing '{spec.pairing}'")
        self.spec = spec
        self.interleaved = spec.pairing == "interleaved"
        self.rotary_dim = spec.head_dim if getattr(spec, "rotary_dim", None) is None else spec.rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= spec.head_dim:
            raise Unsupported(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        self.inv_freq = inverse_frequencies(self.rotary_dim, spec.theta, spec.scaling_dict)
        self.table = None

    def prepare(self, max_positions, device):
        n = min(max_positions, self.spec.max_positions)
        if self.table is not None and self.table.shape[0] >= n and self.table.device == torch.device(device):
            return
        angle = torch.arange(n, dtype=torch.float64)[:, None] * self.inv_freq[None, :]
        table = (torch.cat([angle.cos(), angle.sin()], dim=1) * table_magnitude(self.spec.scaling_dict)).to(torch.float32)
        self.table = table.to(device).contiguous()


register_position("rope", Rope)
