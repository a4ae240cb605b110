"""Rotary position encoding.

The reference computes, per element and per layer, theta_p = 1 / base^(2p/d), the
angle theta_p * pos, and rotates the adjacent pair (2p, 2p+1) of every q and k head
(gpu_kernels.cu:82-112; cpu_decoder.cpp:135-157).  Here the cosines and sines are a
float32 table [positions, rotary_dim / 2], made once from angles taken in float64,
and the rotation is fused with the cache write (``csrc/elementwise.cu``).
``pairing`` = "adjacent" is the reference's; "half" pairs (p, p + rotary_dim / 2).

``scaling`` (the reference has none) stretches the slow pairs for contexts longer than the ``original`` one: with
c(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(c(fast)), 0), hi = min(ceil(c(slow)),
rotary_dim - 1) and r_p = clamp((p - lo) / max(hi - lo, 0.001), 0, 1), pair p turns at
theta_p / factor * r_p + theta_p * (1 - r_p), and every cosine and sine is multiplied by 0.1 ln(factor) + 1.

``scaling`` with ``kind`` = "bands" (keys factor, low, high, original) stretches band by band instead: with the
wavelength l_p = 2 pi / theta_p, pair p keeps theta_p where l_p < original / high, turns at theta_p / factor where
l_p > original / low, and between the two at (1 - s) theta_p / factor + s theta_p with
s = (original / l_p - low) / (high - low); cosines and sines keep their size.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.registry import register_part
from .base import PositionEncoding

PAIRING_CODES = {"adjacent": 0, "half": 1}


@register_part("position", "rotary")
class Rotary(PositionEncoding):
    def __init__(self, head_dim: int, rotary_dim: int, base: float, pairing: str = "adjacent", scaling=None):
        if pairing not in PAIRING_CODES:
            raise ValueError(f"rotary pairing must be one of {sorted(PAIRING_CODES)}, got {pairing!r}")
        if rotary_dim % 2 or not (0 < rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim ({rotary_dim}) must be even and at most head_dim ({head_dim})")
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim
        self.base = float(base)
        self.pairing = pairing
        self.pairing_code = PAIRING_CODES[pairing]
        self.scaling_kind = None
        if scaling is not None:
            self.scaling_kind = scaling.get("kind", "ramp")
            if self.scaling_kind == "bands":
                scaling = {k: float(scaling[k]) for k in ("factor", "original", "low", "high")}
                if min(scaling.values()) <= 0 or scaling["high"] == scaling["low"]:
                    raise ValueError("rotary scaling: factor, original, low and high must be positive, low and high unequal")
            elif self.scaling_kind == "ramp":
                scaling = {k: float(scaling[k]) for k in ("factor", "original", "fast", "slow")}
                if scaling["factor"] <= 0 or scaling["original"] <= 0 or scaling["fast"] <= 0 or scaling["slow"] <= 0:
                    raise ValueError("rotary scaling: factor, original, fast and slow must be positive")
            else:
                raise ValueError(f"rotary scaling: kind must be 'ramp' or 'bands', got {self.scaling_kind!r}")
        self.scaling = scaling
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def prepare(self, max_positions: int, device: torch.device) -> None:
        p = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        inv_freq = 1.0 / torch.pow(torch.tensor(self.base, dtype=torch.float64), 2.0 * p / self.rotary_dim)
        magnitude = 1.0
        if self.scaling_kind == "bands":
            import math
            sc = self.scaling
            wavelength = 2.0 * math.pi / inv_freq
            blend = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
            between = (1.0 - blend) * inv_freq / sc["factor"] + blend * inv_freq
            inv_freq = torch.where(wavelength < sc["original"] / sc["high"], inv_freq,
                                   torch.where(wavelength > sc["original"] / sc["low"], inv_freq / sc["factor"], between))
        elif self.scaling is not None:
            import math
            sc = self.scaling
            turns = lambda t: self.rotary_dim * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(self.base))
            lo = max(math.floor(turns(sc["fast"])), 0)
            hi = min(math.ceil(turns(sc["slow"])), self.rotary_dim - 1)
            ramp = torch.clamp((p - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            inv_freq = inv_freq / sc["factor"] * ramp + inv_freq * (1.0 - ramp)
            magnitude = 0.1 * math.log(sc["factor"]) + 1.0
        angle = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.cos = (angle.cos() * magnitude).to(torch.float32).to(device).contiguous()
        self.sin = (angle.sin() * magnitude).to(torch.float32).to(device).contiguous()
