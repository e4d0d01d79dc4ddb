"""Position encodings."""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import PositionEncoding, Runtime


def rope_inv_freqs(head_dim: int, theta: float, rotary_dim: int | None = None) -> torch.Tensor:
    """``theta^(-2i/rotary_dim)`` for i < rotary_dim/2 as 32-bit floats
    (src/forward/cpu.rs:1057-1061).  Each entry is computed in double precision and rounded
    once, so the table does not depend on a platform's single-precision ``powf``; the table is
    built on the host and the kernels only index it, as the reference does
    (src/forward/gpu.rs:215-219)."""
    rd = head_dim if rotary_dim is None else rotary_dim
    return torch.tensor([float(theta) ** (-2.0 * i / rd) for i in range(rd // 2)],
                        dtype=torch.float64).to(torch.float32)


class RotaryNeoX(PositionEncoding):
    """Split-half rotary embedding: pair ``(i, i + rotary_dim/2)`` of every query and key head
    is rotated by the 32-bit angle ``position * inv_freq[i]`` (src/forward/cpu.rs:1094-1113)."""

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim must be even and in 2..head_dim, got {self.rotary_dim}")
        self._table: torch.Tensor | None = None

    def rotary(self, rt: Runtime):
        if self._table is None or self._table.device != rt.device:
            self._table = rope_inv_freqs(self.head_dim, self.theta, self.rotary_dim).to(rt.device)
        return self._table, self.rotary_dim


class RotaryInterleaved(RotaryNeoX):
    """The same rotation on neighbouring pairs ``(2i, 2i + 1)`` of every head."""

    interleaved = True


class NoPositionEncoding(PositionEncoding):
    """Keys and queries are used as projected."""


register_part("position", "rope_neox", RotaryNeoX)
register_part("position", "rope_interleaved", RotaryInterleaved)
register_part("position", "none", NoPositionEncoding)
