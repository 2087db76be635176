"""Attention over the paged cache: which kernel runs, by dtype, head size and step shape."""
from __future__ import annotations

from . import ops


def attention(qkv, cache_layer, out, ctx, *, n_heads, n_kv_heads, head_dim, scale, window=0):
    """out[t] = softmax(q_t K^T * scale) V over the keys 0..pos(t) of t's slot.  q is the
    leading n_heads*head_dim columns of `qkv`, already rotated."""
    return ops.attention_generic(
        qkv, qkv.shape[1], cache_layer.k, cache_layer.v, ctx.page_table, ctx.token_pos, ctx.token_seq,
        ctx.seq_slot, out, n_tokens=qkv.shape[0], n_heads=n_heads, n_kv_heads=n_kv_heads,
        head_dim=head_dim, page_size=ctx.page_size, scale=scale, window=window)
