"""SwiGLU feed-forward (mlp.rs:31-46): down( silu(gate x) * (up x) ), no biases."""
from __future__ import annotations

import torch

from ..kernels import linear
from .base import FeedForward
from .registry import register
from .spec import TensorSpec


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, *, intermediate_size: int, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.intermediate_size = intermediate_size
        self.w_gate = self.w_up = self.w_down = None

    def tensor_specs(self):
        i, h = self.intermediate_size, self.hidden_size
        return {
            "gate_proj.weight": TensorSpec((i, h)),
            "up_proj.weight": TensorSpec((i, h)),
            "down_proj.weight": TensorSpec((h, i)),
        }

    def set_tensors(self, tensors):
        self.w_gate = linear.Weight(tensors["gate_proj.weight"])
        self.w_up = linear.Weight(tensors["up_proj.weight"])
        self.w_down = linear.Weight(tensors["down_proj.weight"])

    def get_tensors(self):
        return {"gate_proj.weight": self.w_gate.t, "up_proj.weight": self.w_up.t, "down_proj.weight": self.w_down.t}

    def forward(self, x, residual, ctx):
        act = ctx.buffer("ffn_act", (x.shape[0], self.intermediate_size), self.dtype)
        # gate and up in one pass over x, SiLU-gate in the epilogue (mlp.rs:35-43)
        linear.gated(x, self.w_gate, self.w_up, act, ctx)
        # down projection added onto the residual stream (mlp.rs:45, transformer.rs:47)
        linear.into_residual(act, self.w_down, residual, ctx)
