"""RMSNorm, with eps as a parameter (rmsnorm.rs:4-29, math.rs:237-256)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm
from .registry import register
from .spec import TensorSpec


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """y = x * (1 / sqrt(mean(x^2) + eps)) * weight; statistics in float32.  The weight
    multiplies directly (no 1 + w)."""

    def __init__(self, *, eps: float, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.eps = float(eps)
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.hidden_size,), role="vector", init="ones")}

    def set_tensors(self, tensors):
        self.weight = tensors["weight"]

    def get_tensors(self):
        return {"weight": self.weight}

    def forward(self, x, out, rows=None):
        return ops.rmsnorm(x, self.weight, self.eps, out, rows)
