"""Rotary position encoding, rotate-half: dim i pairs with i + rotary_dim/2.

angle = position · inv_freq_i with inv_freq_i = 1 / θ^(2i/rotary_dim), all in 32-bit
(crates/spissa-runtime/src/rotary.rs:454-465); the rotation itself happens in the
kernel that writes the cache (rotary.rs:98-123, :467-481).

``scaling`` of type ``llama3`` rescales the frequency table once (not in the
reference, which drops it: crates/spissa-import/src/safetensors.rs:163-175). With
λ = 2π/inv_freq: λ > n0/low ⇒ inv_freq/factor; λ < n0/high ⇒ unchanged; between,
(1−s)·inv_freq/factor + s·inv_freq with s = (n0/λ − low)/(high − low).
``linear`` divides every frequency by ``factor``.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from .registry import register_part


def rotary_inv_freq(theta: float, rotary_dim: int, scaling: dict | None) -> torch.Tensor:
    """The float32 frequency table [rotary_dim/2], computed on the host in 32-bit."""
    if rotary_dim <= 0 or rotary_dim % 2:
        raise ValueError(f"rotary_dim must be a positive even number, got {rotary_dim}")
    exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / float(rotary_dim)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    if not scaling:
        return inv_freq
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return inv_freq
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv_freq / factor
    if kind == "llama3":
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        n0 = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / inv_freq
        smooth = (n0 / wavelen - low) / (high - low)
        blended = (1.0 - smooth) * inv_freq / factor + smooth * inv_freq
        out = torch.where(wavelen > n0 / low, inv_freq / factor, inv_freq)
        medium = (wavelen <= n0 / low) & (wavelen >= n0 / high)
        return torch.where(medium, blended, out).to(torch.float32)
    raise ValueError(f"unsupported rope scaling type {kind!r}")


@register_part("position", "rotary")
class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, theta: float, rotary_dim: int, scaling: dict | None = None, prefix: str = ""):
        super().__init__(prefix)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim)
        self.scaling = dict(scaling) if scaling else None
        self.inv_freq_host = rotary_inv_freq(self.theta, self.rotary_dim, self.scaling)
        self.inv_freq = None

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.inv_freq = self.inv_freq_host.to(rt.device)

    def rotary(self):
        """(frequency table on the device, rotary_dim) for the fused rotate-and-store kernel."""
        return self.inv_freq, self.rotary_dim
