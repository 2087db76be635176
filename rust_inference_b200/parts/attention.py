"""Grouped-query attention over the cache (attention.rs:54-124)."""
from __future__ import annotations

import math

import torch

from ..cache.sequence_cache import KVRequest
from ..kernels import linear, attention as attn_kernels
from .base import Mixer
from .registry import register, lookup
from .spec import TensorSpec, PartSpec


@register("mixer", "gqa_attention")
class GQAttention(Mixer):
    """q, k, v projections with optional biases (attention.rs:66-76), the position encoding
    on q and k fused with the cache write (:78-90), attention of every new token over the
    keys 0..position of its slot with scale 1/sqrt(head_dim) (:95-121), query head h reading
    kv head h / (heads / kv heads) (:37, :96), and the output projection without bias added
    onto the residual stream (:123, transformer.rs:38-39)."""

    def __init__(self, *, n_heads: int, n_kv_heads: int, head_dim: int, qkv_bias: bool,
                 position: PartSpec, window: int | None = None, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.q_dim, self.kv_dim = n_heads * head_dim, n_kv_heads * head_dim
        self.qkv_bias = bool(qkv_bias)
        self.window = window
        self.scale = 1.0 / math.sqrt(float(head_dim))
        self.position = lookup("position", position.kind)(
            hidden_size=hidden_size, dtype=dtype, device=device, **position.params)
        self.w_qkv = self.b_qkv = self.w_o = None

    def tensor_specs(self):
        h = self.hidden_size
        specs = {
            "q_proj.weight": TensorSpec((self.q_dim, h)),
            "k_proj.weight": TensorSpec((self.kv_dim, h)),
            "v_proj.weight": TensorSpec((self.kv_dim, h)),
            "o_proj.weight": TensorSpec((h, self.q_dim)),
        }
        if self.qkv_bias:
            specs["q_proj.bias"] = TensorSpec((self.q_dim,), role="vector")
            specs["k_proj.bias"] = TensorSpec((self.kv_dim,), role="vector")
            specs["v_proj.bias"] = TensorSpec((self.kv_dim,), role="vector")
        return specs

    def set_tensors(self, tensors):
        # one matrix for the three projections: one pass over x
        self.w_qkv = linear.Weight(torch.cat(
            [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0))
        if self.qkv_bias:
            self.b_qkv = torch.cat(
                [tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]], dim=0).contiguous()
        self.w_o = linear.Weight(tensors["o_proj.weight"])

    def get_tensors(self):
        q, kv = self.q_dim, self.kv_dim
        w = self.w_qkv.t
        out = {"q_proj.weight": w[:q], "k_proj.weight": w[q:q + kv], "v_proj.weight": w[q + kv:],
               "o_proj.weight": self.w_o.t}
        if self.qkv_bias:
            b = self.b_qkv
            out.update({"q_proj.bias": b[:q], "k_proj.bias": b[q:q + kv], "v_proj.bias": b[q + kv:]})
        return out

    def prepare(self, max_positions):
        self.position.prepare(max_positions)

    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, x, residual, ctx, cache_layer, writes_cache):
        n = x.shape[0]
        width = self.q_dim + 2 * self.kv_dim
        from_acc = getattr(self.position, "apply_and_store_from_accumulators", None)
        if from_acc is not None and linear.wants_split(x, self.w_qkv):
            # a small step: the projection is split over K into float32 accumulators, and the
            # position encoding adds the bias, rotates and stores from there
            acc = ctx.zeroed_buffer("qkv_acc", (n, width), torch.float32)
            linear.accumulate_split(x, self.w_qkv, acc, ctx)
            qkv = ctx.buffer("q_rot", (n, self.q_dim), self.dtype)
            from_acc(acc, self.b_qkv, qkv, ctx, cache_layer, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                     head_dim=self.head_dim, write_kv=writes_cache)
        else:
            qkv = ctx.buffer("qkv", (n, width), self.dtype)
            linear.project(x, self.w_qkv, qkv, ctx, bias=self.b_qkv)
            self.position.apply_and_store(qkv, ctx, cache_layer, n_heads=self.n_heads,
                                          n_kv_heads=self.n_kv_heads, head_dim=self.head_dim,
                                          write_kv=writes_cache)
        mixed = ctx.buffer("attn_out", (n, self.q_dim), self.dtype)
        attn_kernels.attention(qkv, cache_layer, mixed, ctx, n_heads=self.n_heads,
                               n_kv_heads=self.n_kv_heads, head_dim=self.head_dim, scale=self.scale,
                               window=self.window or 0)
        linear.into_residual(mixed, self.w_o, residual, ctx)
