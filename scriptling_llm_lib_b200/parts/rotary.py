"""Rotary position encoding: the frequency table, its rescaling, and the rotation of Q and K.

f_i = 1 / theta^(2i / rotary_dim), i < rotary_dim/2; the pair i of a head is rotated by the angle
f_i * position; dimensions past rotary_dim are left alone (model_f32.go:252-260,
float32_ops.go:174-188). The reference pairs adjacent dimensions (2i, 2i+1) ("interleaved"); the
half-split pairing (i, i + rotary_dim/2) is what safetensors checkpoints of the family expect.
The reference knows no frequency rescaling; `llama3` and `linear` rewrite the table on the host.
Angles, cosines and sines are computed on the host in float64 and stored as float32 pairs. The
encoding only owns the table: the mixer's kernels rotate by it (and store keys and values, which
is the mixer's business: V is never rotated, model_f32.go:445-448).
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import POSITION_ENCODINGS, PositionEncoding


def inverse_frequencies(rotary_dim: int, theta: float, scaling=None) -> np.ndarray:
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    f = 1.0 / np.power(float(theta), 2.0 * i / rotary_dim)
    if scaling is None or scaling.rope_type == "default":
        return f
    if scaling.rope_type == "linear":
        return f / scaling.factor
    if scaling.rope_type == "llama3":
        lo_wavelen = scaling.original_max_position_embeddings / scaling.low_freq_factor
        hi_wavelen = scaling.original_max_position_embeddings / scaling.high_freq_factor
        wavelen = 2.0 * math.pi / f
        smooth = (scaling.original_max_position_embeddings / wavelen - scaling.low_freq_factor) / (
            scaling.high_freq_factor - scaling.low_freq_factor)
        blended = (1.0 - smooth) * f / scaling.factor + smooth * f
        return np.where(wavelen > lo_wavelen, f / scaling.factor, np.where(wavelen < hi_wavelen, f, blended))
    raise ValueError(f"unknown rope scaling {scaling.rope_type!r}")


class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, rotary_dim: int, theta: float, scaling=None, pairing: str = "half"):
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rope pairing {pairing!r}; known: half, interleaved")
        if rotary_dim % 2 or not 2 <= rotary_dim <= head_dim:
            raise ValueError(f"rotary width {rotary_dim} must be even and within 2..{head_dim}")
        self.head_dim, self.rotary_dim, self.theta, self.scaling, self.pairing = head_dim, rotary_dim, theta, scaling, pairing
        self.inv_freq = inverse_frequencies(rotary_dim, theta, scaling)
        self.cos_sin: torch.Tensor | None = None     # [positions, rotary_dim/2, 2] float32

    def prepare(self, max_positions: int, device) -> None:
        if self.cos_sin is not None and self.cos_sin.shape[0] >= max_positions and self.cos_sin.device == torch.device(device):
            return
        ang = np.arange(max_positions, dtype=np.float64)[:, None] * self.inv_freq[None, :]
        table = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)
        self.cos_sin = torch.from_numpy(table).to(device).contiguous()

    @property
    def max_positions(self) -> int:
        return 0 if self.cos_sin is None else self.cos_sin.shape[0]

    def rotation(self):
        """(table [positions, rotary_dim / 2, 2] of (cos, sin), rotary width, interleaved pairing)."""
        return self.cos_sin, self.rotary_dim, self.pairing == "interleaved"


POSITION_ENCODINGS.register("rotary", RotaryEncoding)
