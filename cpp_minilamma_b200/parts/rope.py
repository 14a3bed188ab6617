"""Rotary position encoding: host-built cos/sin tables.

Pair i of a head rotates by angle pos * f_i with f_i = theta^(-2i/d)
(src/ops.cc:200-205).  The reference evaluates pow/cos/sin per token (in double on the
CPU, in float on the GPU: src/cuda_ops.cu:254-299); here the table is computed once in
double and stored as float32 [max_positions, d/2], so every kernel and every position
sees the same, correctly rounded angles.

`scaling` of type llama3 changes the frequencies once (the reference has no rope
scaling): with L0 = original_max_position_embeddings and wavelength lam = 2 pi / f,
f is kept when lam < L0 / high_freq_factor, divided by `factor` when
lam > L0 / low_freq_factor, and otherwise blended with
s = (L0 / lam - low) / (high - low):  f' = (1 - s) f / factor + s f.

`interleaved` selects the pairing: True pairs (2i, 2i+1) (the reference's Normal type),
False pairs (i, i + d/2) (its NeoX type), src/ops.cc:206-210.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import numpy as np
import torch

from .base import BuildContext, PositionEncoding, register_part


def inverse_frequencies(head_dim: int, theta: float, scaling: Optional[Dict[str, Any]]) -> np.ndarray:
    half = head_dim // 2
    freqs = np.power(float(theta), -2.0 * np.arange(half, dtype=np.float64) / head_dim)
    if not scaling:
        return freqs
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    wavelength = 2.0 * math.pi / freqs
    smooth = (original / wavelength - low) / (high - low)
    blended = (1.0 - smooth) * freqs / factor + smooth * freqs
    return np.where(wavelength < original / high, freqs,
                    np.where(wavelength > original / low, freqs / factor, blended))


class RotaryEncoding(PositionEncoding):
    """params: head_dim, theta, scaling (dict or None), interleaved."""

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.head_dim = int(params["head_dim"])
        self.interleaved = bool(params.get("interleaved", False))
        if self.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {self.head_dim}")
        freqs = inverse_frequencies(self.head_dim, float(params["theta"]), params.get("scaling"))
        angles = np.arange(ctx.max_positions, dtype=np.float64)[:, None] * freqs[None, :]
        self.cos = torch.from_numpy(np.cos(angles).astype(np.float32)).to(ctx.device)
        self.sin = torch.from_numpy(np.sin(angles).astype(np.float32)).to(ctx.device)

    def tables(self):
        return self.cos, self.sin


class NoPositionEncoding(PositionEncoding):
    """Positions are not encoded; q and k pass through unrotated."""

    interleaved = False

    def tables(self):
        return None, None


def shared_position_encoding(spec, ctx: BuildContext):
    """Layers with equal parameters share one table."""
    from .base import build_part
    key = ("position_encoding", spec.kind, repr(sorted(spec.params.items(), key=lambda kv: kv[0])))
    if key not in ctx.shared:
        ctx.shared[key] = build_part("position_encoding", spec, ctx)
    return ctx.shared[key]


register_part("position_encoding", "rotary", RotaryEncoding)
register_part("position_encoding", "none", NoPositionEncoding)
