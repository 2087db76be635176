"""The output head: final norm, then logits = W h in float32, on the wanted rows only
(transformer.rs:89, :97).  The matrix is the embedding's when the model ties them: the same
storage, where the reference clones it (model.rs:221-226)."""
from __future__ import annotations

import torch

from ..kernels import linear
from .base import Head
from .registry import lookup, register
from .spec import PartSpec, TensorSpec


@register("head", "linear_head")
class LinearHead(Head):
    def __init__(self, *, vocab_size: int, norm: PartSpec, tied: bool, weight_prefix: str | None = "lm_head.",
                 hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.vocab_size = vocab_size
        self.wants_tie = bool(tied)
        self.weight_prefix = weight_prefix
        self.norm_prefix = norm.prefix
        self.norm = lookup("norm", norm.kind)(hidden_size=hidden_size, dtype=dtype, device=device, **norm.params)
        self.weight = None

    def tensor_specs(self):
        specs = {self.norm_prefix + local: ts for local, ts in self.norm.tensor_specs().items()}
        if not self.wants_tie:
            specs[self.weight_prefix + "weight"] = TensorSpec((self.vocab_size, self.hidden_size))
        return specs

    def set_tensors(self, tensors):
        n = len(self.norm_prefix)
        self.norm.set_tensors({name[n:]: t for name, t in tensors.items() if name.startswith(self.norm_prefix)
                               and name[n:] in self.norm.tensor_specs()})
        if not self.wants_tie:
            self.weight = linear.Weight(tensors[self.weight_prefix + "weight"])

    def get_tensors(self):
        out = {self.norm_prefix + local: t for local, t in self.norm.get_tensors().items()}
        if not self.wants_tie:
            out[self.weight_prefix + "weight"] = self.weight.t
        return out

    def tie(self, table):
        self.weight = linear.Weight(table)            # the same storage, no copy

    def prepare(self, max_positions):
        self.norm.prepare(max_positions)

    def matrix_bytes(self):
        return self.weight.t.numel() * self.weight.t.element_size()

    def normalised(self, residual, rows):
        out = torch.empty((rows.numel(), self.hidden_size), dtype=self.dtype, device=residual.device)
        self.norm.forward(residual, out, rows=rows)
        return out

    def forward(self, residual, ctx, logits_out=None):
        normed = ctx.buffer("head_in", (ctx.n_logit_rows, self.hidden_size), self.dtype)
        self.norm.forward(residual, normed, rows=ctx.logit_rows)
        if logits_out is None:
            logits_out = torch.empty((ctx.n_logit_rows, self.vocab_size), dtype=torch.float32, device=residual.device)
        linear.logits(normed, self.weight, logits_out, ctx)
        return logits_out
