"""Attention over the paged cache: which kernel runs, by dtype, head size and step shape.

  bfloat16, head_dim 64 or 128   one token per sequence: split-K over runs of pages
                                 (`attention_mma`); otherwise the tcgen05 flash-style causal
                                 kernel (`attention_tcgen05`), with the mma.sync one behind it
  anything else                  the generic kernel (`attention_generic`): any head size, any
                                 dtype, float32 arithmetic
"""
from __future__ import annotations

import os

import torch

from . import ops

N_SMS = 148
# RI_B200_PREFILL_ATTENTION=mma keeps the mma.sync prefill kernel (for comparisons)
_PREFILL = os.environ.get("RI_B200_PREFILL_ATTENTION", "tcgen05")
# RI_B200_DECODE_ATTENTION=cp_async / tma forces one of the two decode kernels (default: by batch size)
_DECODE = os.environ.get("RI_B200_DECODE_ATTENTION", "auto")


def decode_splits(n_seqs: int, n_kv_heads: int, max_seq_len: int, page_size: int) -> int:
    """Runs of pages per (sequence, kv head): as many CTAs as are resident at once (two per SM),
    never more, so the grid is one wave; never more runs than the longest sequence has pages.
    Depends on the batch size and the cache geometry only, so a captured step keeps its grid."""
    pairs = max(1, n_seqs * n_kv_heads)
    want = (2 * N_SMS) // pairs
    return max(1, min(want, 32, -(-max_seq_len // page_size)))


def attention(qkv, cache_layer, out, ctx, *, n_heads, n_kv_heads, head_dim, scale, window=0):
    """out[t] = softmax(q_t K^T * scale) V over the keys 0..pos(t) of t's slot.  q is the
    leading n_heads*head_dim columns of `qkv`, already rotated."""
    q_ld = qkv.shape[1]
    if qkv.dtype == torch.bfloat16:
        decode = ctx.all_single
        if ops.attention_mma_supports(head_dim, ctx.page_size, n_heads, n_kv_heads, decode):
            if decode:
                max_len = ctx.page_table.shape[1] * ctx.page_size
                splits = decode_splits(ctx.n_seqs, n_kv_heads, max_len, ctx.page_size)
                part_o = part_ml = None
                if splits > 1:
                    part_o = ctx.buffer("attn_part_o", (ctx.n_seqs * n_heads * splits * head_dim,), torch.float32)
                    part_ml = ctx.buffer("attn_part_ml", (ctx.n_seqs * n_heads * splits * 2,), torch.float32)
                from . import attention_tc
                # Large batches stream many pages per CTA: the TMA ring keeps more of them in flight
                # (batch 64, 1,024 positions: 26.7 us against 40.9 us).  Small batches are cut into
                # short runs that are latency bound, where the cp.async kernel is about 1 us quicker.
                use_tma = _DECODE == "tma" or (_DECODE == "auto" and splits == 1)
                decode_fn = attention_tc.decode if use_tma else ops.attention_decode
                return decode_fn(
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
