"""Python face of the tcgen05 + TMA contraction kernel (bf16 operands, float32 accumulate)."""
from __future__ import annotations


def supports(x, w) -> bool:
    return False


def gemm(x, w, out, mode, ctx, bias=None, w2=None):
    raise NotImplementedError
