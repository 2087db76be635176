"""The token embedding: a row of the table per token, widened to float32 (transformer.rs:74-75)."""
from __future__ import annotations

from ..kernels import ops
from .base import Embedding
from .registry import register
from .spec import TensorSpec


@register("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, *, vocab_size: int, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.vocab_size = vocab_size
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def set_tensors(self, tensors):
        self.weight = tensors["weight"]

    def get_tensors(self):
        return {"weight": self.weight}

    def table(self):
        return self.weight

    def forward(self, ctx, residual):
        ops.embed_gather(self.weight, ctx.token_ids, residual)
