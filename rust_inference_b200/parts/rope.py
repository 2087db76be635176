"""Rotary position encoding, with base and pairing as parameters (rope.rs:42-98)."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import PositionEncoding
from .registry import register

_STYLES = {"half": 0, "interleaved": 1}


def rope_tables(head_dim: int, base: float, n_positions: int):
    """cos, sin as float32 [n_positions, head_dim/2], built the way rope.rs:47-55 does:
    exponent = 2i/dim, theta = 1/base^exponent and angle = pos*theta are 32-bit numbers
    (the power is taken in float64 and rounded once); cos and sin are taken of the 32-bit
    angle in float64 and rounded once."""
    half = head_dim // 2
    exponent = (2 * np.arange(half)).astype(np.float32) / np.float32(head_dim)
    theta = (1.0 / np.power(np.float64(np.float32(base)), exponent.astype(np.float64))).astype(np.float32)
    pos = np.arange(n_positions, dtype=np.float32)
    angle = (pos[:, None] * theta[None, :]).astype(np.float32)
    cos = np.cos(angle.astype(np.float64)).astype(np.float32)
    sin = np.sin(angle.astype(np.float64)).astype(np.float32)
    return cos, sin


@register("position", "rope")
class RotaryEncoding(PositionEncoding):
    """Rotates every q head and every k head by the angles of the token's absolute
    position (attention.rs:78-87); v is not rotated.  style "interleaved" pairs (2i, 2i+1)
    as rope.rs:92-96 does; "half" pairs (i, i + dim/2)."""

    def __init__(self, *, head_dim: int, base: float, style: str = "half", hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if style not in _STYLES:
            raise ValueError(f"rope style must be one of {sorted(_STYLES)}, found {style!r}")
        if head_dim % 2:
            raise ValueError(f"rope needs an even head_dim, found {head_dim}")
        self.head_dim = head_dim
        self.base = float(base)
        self.style = _STYLES[style]
        self.cos = self.sin = None

    def prepare(self, max_positions: int) -> None:
        if self.cos is None or self.cos.shape[0] < max_positions:
            cos, sin = rope_tables(self.head_dim, self.base, max_positions)
            self.cos = torch.from_numpy(cos).to(self.device)
            self.sin = torch.from_numpy(sin).to(self.device)

    def apply_and_store(self, qkv, ctx, cache_layer, *, n_heads, n_kv_heads, head_dim, write_kv):
        if self.cos is None or self.cos.shape[0] < ctx.max_len:
            raise RuntimeError("rope tables do not cover the step's positions; call prepare() first")
        ops.rope_cache_write(qkv, self.cos, self.sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot,
                             ctx.page_table, cache_layer.k, cache_layer.v, n_heads=n_heads,
                             n_kv_heads=n_kv_heads, head_dim=head_dim, page_size=ctx.page_size,
                             style=self.style, write_kv=write_kv)

    def apply_and_store_from_accumulators(self, acc, bias, q_out, ctx, cache_layer, *, n_heads, n_kv_heads,
                                          head_dim, write_kv):
        """The same from float32 accumulators of a K-split projection (bias not yet added): q goes
        to q_out, and `acc` is left zeroed."""
        if self.cos is None or self.cos.shape[0] < ctx.max_len:
            raise RuntimeError("rope tables do not cover the step's positions; call prepare() first")
        ops.rope_cache_write_acc(acc, bias, q_out, self.cos, self.sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot,
                                 ctx.page_table, cache_layer.k, cache_layer.v, n_heads=n_heads,
                                 n_kv_heads=n_kv_heads, head_dim=head_dim, page_size=ctx.page_size,
                                 style=self.style, write_kv=write_kv)
