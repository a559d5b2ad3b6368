"""Position encodings of attention mixers.

"rope": rotation of pairs of q and k elements by position-dependent angles
(src/kernels/rotary_embedding.cu:18-33).  The angle of pair j at position p is
p / theta^(2j / rotary_dim), evaluated in float as the reference's table is
(src/model/qwen.cpp:119-128: ``pos / powf(theta, 2i/d)``).  The divisors are
computed once on the host; the kernel divides and calls sincosf per element, so
no table grows with the context length.  ``pairing`` "half" pairs element j with
j + rotary_dim/2 (what the reference does), "interleaved" pairs 2j with 2j+1.
``rotary_dim`` below the head size leaves the rest of each head unrotated.

"none": no position information is added.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .base import PositionEncoding, register_position_encoding

PAIRINGS = {"half": 0, "interleaved": 1}


@register_position_encoding("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, theta: float, rotary_dim: int, pairing: str = "half", dtype=None, device=None):
        if pairing not in PAIRINGS:
            raise ValueError(f"rope pairing {pairing!r}; known: {sorted(PAIRINGS)}")
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rope rotary_dim {rotary_dim} must be positive and even")
        if not theta > 0:
            raise ValueError(f"rope theta {theta} must be positive")
        self.theta, self.rotary_dim, self.pairing = float(theta), rotary_dim, pairing
        j = np.arange(rotary_dim // 2, dtype=np.float32)
        exponent = (np.float32(2.0) * j) / np.float32(rotary_dim)
        # theta and the exponent as the reference has them, in float (src/model/qwen.cpp:124); the power itself in
        # double and then rounded, so that every host that computes it gets the same float (powf differs from one
        # library to the next in the last bit, which is enough to move a sampled token)
        denom = np.power(np.float64(np.float32(theta)), exponent.astype(np.float64)).astype(np.float32)
        self.denom = torch.from_numpy(denom).to(device)

    def fused(self) -> Optional[dict]:
        return {"rotary_dim": self.rotary_dim, "pairing": PAIRINGS[self.pairing], "denom": self.denom}


def rescale_by_wavelength(freq: np.ndarray, factor: float, low: float, high: float, original: float) -> np.ndarray:
    """Frequencies (float64) rescaled by wavelength l = 2 pi / f, as contexts are stretched beyond ``original`` positions:
    short waves (l < original / high) stay, long ones (l > original / low) are divided by ``factor``, and between the two
    the frequency is (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    if not (factor > 0 and original > 0 and high > low >= 0):
        raise ValueError(f"frequency scaling: factor {factor}, low {low} < high {high}, original {original}")
    wavelength = 2.0 * np.pi / freq
    s = (original / wavelength - low) / (high - low)
    between = (1.0 - s) * freq / factor + s * freq
    return np.where(wavelength < original / high, freq, np.where(wavelength > original / low, freq / factor, between))


@register_position_encoding("scaled_rope")
class ScaledRotaryEmbedding(RotaryEmbedding):
    """"rope" whose frequencies f_i = theta^(-2i / rotary_dim) are rescaled by wavelength (``scaling``: None, or
    {"factor", "low", "high", "original"}; rescale_by_wavelength).  The frequencies are computed in double and rounded
    once; ``inv_freq`` (float32 [rotary_dim / 2]) is what a kernel multiplies a position by, ``denom`` its reciprocal
    for kernels that divide."""

    def __init__(self, theta: float, rotary_dim: int, pairing: str = "half", scaling: Optional[dict] = None, dtype=None, device=None):
        super().__init__(theta, rotary_dim, pairing, dtype=dtype, device=device)
        i = np.arange(rotary_dim // 2, dtype=np.float64)
        freq = np.power(float(theta), -2.0 * i / rotary_dim)
        if scaling is not None:
            missing = [k for k in ("factor", "low", "high", "original") if k not in scaling]
            if missing:
                raise ValueError(f"scaled_rope: scaling lacks {missing}")
            freq = rescale_by_wavelength(freq, float(scaling["factor"]), float(scaling["low"]), float(scaling["high"]),
                                         float(scaling["original"]))
        self.scaling = dict(scaling) if scaling is not None else None
        self.inv_freq = torch.from_numpy(freq.astype(np.float32)).to(device)
        self.denom = torch.from_numpy((1.0 / freq).astype(np.float32)).to(device)


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    def __init__(self, dtype=None, device=None):
        pass

    def fused(self) -> Optional[dict]:
        return {"rotary_dim": 0, "pairing": 0, "denom": None}
