"""The contractions of the decoder, out = x @ W^T, each with its epilogue fused.

Which kernel runs is decided here, by dtype and shape:
  float32   always the FFMA kernel (`gemm_simt`): no tensor-core mode touches a 32-bit run;
  bfloat16  the tcgen05 kernel (`gemm_tcgen05`) when the shape meets its alignment rule,
            else the FFMA kernel on bf16 operands.  Either way accumulation is float32.
"""
from __future__ import annotations

import torch

from . import ops


class Weight:
    """A weight matrix [out, in] (row-major over `in`, as quant.rs:45-50 holds it) plus
    whatever a kernel wants to keep beside it (tensor-map handles)."""

    __slots__ = ("t", "n", "k", "tc")

    def __init__(self, t: torch.Tensor):
        self.t = t.contiguous()
        self.n, self.k = self.t.shape
        self.tc = None


def _use_tensor_cores(x: torch.Tensor, w: Weight) -> bool:
    if x.dtype != torch.bfloat16:
        return False
    from . import tcgen05
    return tcgen05.supports(x, w)


def project(x, w: Weight, out, ctx, bias=None):
    """out<run dtype> = x W^T + bias."""
    if _use_tensor_cores(x, w):
        from . import tcgen05
        return tcgen05.gemm(x, w, out, ops.EPI_STORE, ctx, bias=bias)
    return ops.gemm_simt(x, w.t, out, ops.EPI_STORE, bias=bias)


def logits(x, w: Weight, out, ctx):
    """out<float32> = x W^T."""
    if _use_tensor_cores(x, w):
        from . import tcgen05
        return tcgen05.gemm(x, w, out, ops.EPI_STORE_F32, ctx)
    return ops.gemm_simt(x, w.t, out, ops.EPI_STORE_F32)


def into_residual(x, w: Weight, residual, ctx):
    """residual<float32> += x W^T."""
    if _use_tensor_cores(x, w):
        from . import tcgen05
        return tcgen05.gemm(x, w, residual, ops.EPI_RESIDUAL, ctx)
    return ops.gemm_simt(x, w.t, residual, ops.EPI_RESIDUAL)


def gated(x, w_gate: Weight, w_up: Weight, out, ctx):
    """out<run dtype> = silu(x Wg^T) * (x Wu^T)."""
    if _use_tensor_cores(x, w_gate):
        from . import tcgen05
        return tcgen05.gemm(x, w_gate, out, ops.EPI_SILU_MUL, ctx, w2=w_up)
    return ops.gemm_simt(x, w_gate.t, out, ops.EPI_SILU_MUL, w2=w_up.t)


def accumulate_split(x, w: Weight, acc, ctx) -> bool:
    """acc<float32> += x W^T with K split over enough CTAs to fill the GPU, if the tensor-core
    kernel takes the shape (returns False otherwise and does nothing).  For small steps whose
    output has too few tiles to keep every SM streaming weights."""
    if not _use_tensor_cores(x, w):
        return False
    from . import tcgen05
    tcgen05.gemm(x, w, acc, ops.EPI_RESIDUAL, ctx)
    return True


# Up to this many tokens a projection that has to leave its result in the run dtype is worth cutting
# over K into float32 accumulators (measured on a 3584-wide model: a whole 256-token step 1.4% faster,
# a 512-token step 2% slower)
SPLIT_MAX_TOKENS = 256


def wants_split(x, w: Weight) -> bool:
    """True for a small step whose projection would otherwise leave most SMs idle."""
    if not _use_tensor_cores(x, w) or x.shape[0] > SPLIT_MAX_TOKENS:
        return False
    from . import tcgen05
    return tcgen05.pick_split(x.shape[0], w.n, w.k) > 1
