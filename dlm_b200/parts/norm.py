"""Normalisation parts."""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import Norm, ParamSpec, Runtime


class RMSNorm(Norm):
    """``out = (x / sqrt(mean(x^2) + eps)) * weight`` with 32-bit statistics
    (src/forward/cpu.rs:934-942); the result is stored in the activation dtype."""

    def __init__(self, size: int, eps: float):
        self.size, self.eps = int(size), float(eps)
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return [ParamSpec("weight", (self.size,), init="norm")]

    def load(self, tensors, rt: Runtime):
        self.weight = rt.vector(tensors["weight"])

    def forward(self, x, rt: Runtime, rows=None, out_dtype=None):
        return rt.ops.rmsnorm(x, self.weight, self.eps, out_dtype or rt.dtype, rows)

    def fusable_rms(self):
        return self.weight, self.eps


register_part("norm", "rmsnorm", RMSNorm)
