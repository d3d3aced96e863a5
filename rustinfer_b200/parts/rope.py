"""Rotary position encoding: the frequency law and the cos/sin tables.

inv_freq f_i = theta^(-2i/rotary_dim); with llama3 scaling each frequency is kept, divided
by `factor`, or blended, by the band its wavelength falls in
(crates/infer-worker/src/models/loader.rs:1543-1571).  Angles pos*f_i are formed in
float64 and the tables are stored fp32 [positions, rotary_dim/2]; RustInfer stores them in
the activation dtype (bf16 in production, :1574-1589), which costs three digits of the
angle for nothing.  The rotation itself (pair i, i+rotary_dim/2) is in the kernel that
also writes keys and values into the cache.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .base import BuildContext, PositionEncoding, register_position


def rope_inv_freq(rotary_dim: int, theta: float, scaling: Optional[dict]) -> List[float]:
    half = rotary_dim // 2
    freqs = [theta ** (-2.0 * i / rotary_dim) for i in range(half)]
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind != "llama3":
            raise ValueError(f"rope scaling of type {kind!r} is not built; known: 'llama3'")
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        long_wave, short_wave = orig / low, orig / high
        for i, f in enumerate(freqs):
            wave = 2.0 * math.pi / f
            if wave < short_wave:
                continue
            if wave > long_wave:
                freqs[i] = f / factor
            else:
                blend = (orig / wave - low) / (high - low)
                freqs[i] = (1.0 - blend) * f / factor + blend * f
    return freqs


@register_position("rope")
class RotaryEncoding(PositionEncoding):
    """params: head_dim, rotary_dim, theta, scaling (dict or None)."""

    def __init__(self, params):
        super().__init__(params)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim") or self.head_dim)
        self.theta = float(params["theta"])
        self.scaling = dict(params["scaling"]) if params.get("scaling") else None
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def tables(self, positions: int):
        """(cos, sin) as float64 CPU tensors [positions, rotary_dim/2]."""
        f = torch.tensor(rope_inv_freq(self.rotary_dim, self.theta, self.scaling), dtype=torch.float64)
        ang = torch.arange(positions, dtype=torch.float64)[:, None] * f[None, :]
        return torch.cos(ang), torch.sin(ang)

    def prepare(self, ctx: BuildContext) -> None:
        super().prepare(ctx)
        c, s = self.tables(ctx.max_model_len)
        self.cos = c.to(torch.float32).to(ctx.device).contiguous()
        self.sin = s.to(torch.float32).to(ctx.device).contiguous()
