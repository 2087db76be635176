"""Attention over the paged cache: which kernel runs, by dtype, head size and step shape.

  bfloat16, head_dim 64 or 128   one token per sequence: split-K over runs of pages
                                 (`attention_mma`); otherwise the tcgen05 flash-style causal
                                 kernel (`attention_tcgen05`), with the mma.sync one behind it
  anything else                  the generic kernel (`attention_generic`): any head size, any
                                 dtype, float32 arithmetic
"""
from __future__ import annotations

import functools
import os

import torch

from . import ops


@functools.lru_cache(maxsize=None)
def _sm_count() -> int:
    """SMs of the current device (148 on a B200)."""
    return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)

# RI_B200_PREFILL_ATTENTION=mma keeps the mma.sync prefill kernel (for comparisons)
_PREFILL = os.environ.get("RI_B200_PREFILL_ATTENTION", "tcgen05")
# RI_B200_DECODE_ATTENTION=cluster / cp_async / tma forces one of the decode kernels (default: by batch size)
_DECODE = os.environ.get("RI_B200_DECODE_ATTENTION", "auto")
CLUSTER_SPLITS = 8     # a thread-block cluster holds at most 8 CTAs portably


def decode_splits(n_seqs: int, n_kv_heads: int, max_seq_len: int, page_size: int, limit: int = 32) -> int:
    """Runs of pages per (sequence, kv head): as many CTAs as are resident at once (two per SM),
    never more, so the grid is one wave; never more runs than the longest sequence has pages.
    Depends on the batch size and the cache geometry only, so a captured step keeps its grid."""
    pairs = max(1, n_seqs * n_kv_heads)
    want = (2 * _sm_count()) // pairs
    if os.environ.get("RI_B200_DECODE_SPLITS"):
        want = int(os.environ["RI_B200_DECODE_SPLITS"])
    return max(1, min(want, limit, -(-max_seq_len // page_size)))


def decode_plan(n_seqs: int, n_kv_heads: int, max_seq_len: int, page_size: int, head_dim: int | None = None):
    """Which decode kernel a step of n_seqs sequences takes, and into how many runs of pages it
    cuts a sequence: ("cluster" | "tma" | "cp_async", splits).  Left to itself it answers "cluster"
    (the TMA-fed kernel with the 2..8 runs of a sequence as one thread-block cluster) while a step's
    sequences x kv heads leave SMs idle, and "tma" (the same kernel, one run per sequence) beyond;
    "cp_async" (pages by cp.async, runs merged through scratch by a second kernel) is only taken
    when RI_B200_DECODE_ATTENTION asks for it: it is the kernel of the allocation-free entry point
    and the comparison for the other two.

    Split runs are merged inside the kernel when the splits of a (sequence, kv head) fit a
    thread-block cluster: no scratch round trip and no second kernel.  With `head_dim` given the
    device is asked how many such clusters it holds at once, and the runs are made fewer until the
    whole step is resident together."""
    if _DECODE in ("auto", "cluster"):
        splits = decode_splits(n_seqs, n_kv_heads, max_seq_len, page_size, CLUSTER_SPLITS)
        if head_dim is not None:
            from . import attention_tc
            while splits >= 2 and attention_tc.decode_cluster_capacity(head_dim, splits) < n_seqs * n_kv_heads:
                splits -= 1
        if splits >= 2:
            return "cluster", splits
    # no clusters (one run per sequence is enough, or the device holds too few): the same kernel, its runs,
    # if any, merged through scratch by a second kernel
    splits = decode_splits(n_seqs, n_kv_heads, max_seq_len, page_size)
    return ("cp_async" if _DECODE == "cp_async" else "tma"), splits


def decode_kernel(name: str):
    if name == "cluster":
        from . import attention_tc
        return attention_tc.decode_cluster
    if name == "tma":
        from . import attention_tc
        return attention_tc.decode
    return ops.attention_decode


def attention(qkv, cache_layer, out, ctx, *, n_heads, n_kv_heads, head_dim, scale, window=0):
    """out[t] = softmax(q_t K^T * scale) V over the keys 0..pos(t) of t's slot.  q is the
    leading n_heads*head_dim columns of `qkv`, already rotated."""
    q_ld = qkv.shape[1]
    if qkv.dtype == torch.bfloat16:
        decode = ctx.all_single
        if ops.attention_mma_supports(head_dim, ctx.page_size, n_heads, n_kv_heads, decode):
            if decode:
                max_len = ctx.page_table.shape[1] * ctx.page_size
                name, splits = decode_plan(ctx.n_seqs, n_kv_heads, max_len, ctx.page_size, head_dim)
                part_o = part_ml = None
                if splits > 1 and name != "cluster":
                    part_o = ctx.buffer("attn_part_o", (ctx.n_seqs * n_heads * splits * head_dim,), torch.float32)
                    part_ml = ctx.buffer("attn_part_ml", (ctx.n_seqs * n_heads * splits * 2,), torch.float32)
                return decode_kernel(name)(
                    qkv, q_ld, cache_layer.k, cache_layer.v, ctx.page_table, ctx.seq_slot, ctx.seq_len,
                    ctx.cu_seqlens, out, n_seqs=ctx.n_seqs, n_heads=n_heads, n_kv_heads=n_kv_heads,
                    head_dim=head_dim, page_size=ctx.page_size, scale=scale, window=window, n_splits=splits,
                    part_o=part_o, part_ml=part_ml)
            from . import attention_tc
            if _PREFILL != "mma" and attention_tc.supports(head_dim, ctx.page_size, n_heads, n_kv_heads, q_ld,
                                                           out.shape[1]):
                return attention_tc.prefill(
                    qkv, cache_layer.k, cache_layer.v, ctx.page_table, ctx.seq_slot, ctx.seq_start, ctx.cu_seqlens,
                    out, n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=n_heads, n_kv_heads=n_kv_heads,
                    head_dim=head_dim, page_size=ctx.page_size, scale=scale, window=window)
            return ops.attention_prefill(
                qkv, q_ld, cache_layer.k, cache_layer.v, ctx.page_table, ctx.seq_slot, ctx.seq_start,
                ctx.cu_seqlens, out, n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=n_heads,
                n_kv_heads=n_kv_heads, head_dim=head_dim, page_size=ctx.page_size, scale=scale, window=window)
    return ops.attention_generic(
        qkv, q_ld, cache_layer.k, cache_layer.v, ctx.page_table, ctx.token_pos, ctx.token_seq,
        ctx.seq_slot, out, n_tokens=qkv.shape[0], n_heads=n_heads, n_kv_heads=n_kv_heads,
        head_dim=head_dim, page_size=ctx.page_size, scale=scale, window=window)
