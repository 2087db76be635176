"""Python face of the tcgen05 prefill attention: tensor maps (kept per buffer) and the call."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import ops
from .build import load
from .ops import _call, _need, _need_cuda, _p, _stream
from .tcgen05 import status_word

_maps: dict = {}


def supports(head_dim: int, page_size: int, n_heads: int, n_kv_heads: int, q_ld: int, out_ld: int) -> bool:
    lib = load("attention_tcgen05")
    return bool(lib.ri_attention_tcgen05_supports(c_int(head_dim), c_int(page_size), c_int(n_heads),
                                                  c_int(n_kv_heads), c_int(q_ld), c_int(out_ld)))


def _map(which: int, t: torch.Tensor, rows: int, cols: int, ld: int) -> torch.Tensor:
    key = (which, t.data_ptr(), rows, cols, ld)
    m = _maps.get(key)
    if m is None:
        if len(_maps) > 8192:
            _maps.clear()
        m = torch.empty(128, dtype=torch.uint8)
        _call("attention_tcgen05", "ri_attention_tcgen05_encode", c_void_p(m.data_ptr()), c_int(which), _p(t),
              c_longlong(rows), c_longlong(cols), c_longlong(ld))
        ops._launches -= 1
        _maps[key] = m
    return m


def prefill(qkv: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, page_table, seq_slot, seq_start,
            cu_seqlens, out: torch.Tensor, *, n_seqs: int, max_new: int, n_heads: int, n_kv_heads: int,
            head_dim: int, page_size: int, scale: float, window: int = 0) -> torch.Tensor:
    """bf16 causal attention of every new token over its slot's keys, on tcgen05.  q is the leading
    n_heads * head_dim columns of `qkv`; kcache / vcache are one layer, [pages, kv heads, 64, head_dim]."""
    _need_cuda(qkv, kcache, vcache, page_table, seq_slot, seq_start, cu_seqlens, out)
    _need(qkv.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
          and qkv.is_contiguous() and kcache.is_contiguous() and vcache.is_contiguous() and out.is_contiguous(),
          "attention_tcgen05: bf16 contiguous tensors only")
    rows = kcache.shape[0] * kcache.shape[1] * kcache.shape[2]
    mq = _map(0, qkv, qkv.shape[0], qkv.shape[1], qkv.shape[1])
    mk = _map(1, kcache, rows, head_dim, head_dim)
    mv = _map(1, vcache, rows, head_dim, head_dim)
    st = status_word()
    _call("attention_tcgen05", "ri_attention_tcgen05_prefill", c_void_p(mq.data_ptr()), c_void_p(mk.data_ptr()),
          c_void_p(mv.data_ptr()), _p(page_table), c_int(page_table.shape[1]), _p(seq_slot), _p(seq_start),
          _p(cu_seqlens), _p(out), c_int(out.shape[1]), c_int(n_seqs), c_int(max_new), c_int(n_heads),
          c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_float(scale), c_int(window),
          c_void_p(st.data_ptr()), _stream())
    return out


def decode(q: torch.Tensor, q_ld: int, kcache: torch.Tensor, vcache: torch.Tensor, page_table, seq_slot, seq_len,
           cu_seqlens, out: torch.Tensor, *, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int,
           page_size: int, scale: float, window: int, n_splits: int, part_o=None, part_ml=None) -> torch.Tensor:
    """Split-K decode attention (one new token per sequence) with the cache pages brought in by TMA
    through a three-stage ring; same arguments and scratch as `ops.attention_decode`."""
    _need_cuda(q, kcache, vcache, page_table, seq_slot, seq_len, cu_seqlens, out, part_o, part_ml)
    _need(q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
          and kcache.is_contiguous() and vcache.is_contiguous(), "attention_decode: bf16 contiguous tensors only")
    if n_splits > 1:
        _need(part_o is not None and part_o.numel() >= n_seqs * n_heads * n_splits * head_dim
              and part_ml is not None and part_ml.numel() >= n_seqs * n_heads * n_splits * 2,
              "attention_decode: scratch too small")
    rows = kcache.shape[0] * kcache.shape[1] * kcache.shape[2]
    mk = _map(1, kcache, rows, head_dim, head_dim)
    mv = _map(1, vcache, rows, head_dim, head_dim)
    st = status_word()
    _call("attention_mma", "ri_attention_decode_tma", c_void_p(mk.data_ptr()), c_void_p(mv.data_ptr()), _p(q),
          c_int(q_ld), _p(page_table), c_int(page_table.shape[1]), _p(seq_slot), _p(seq_len), _p(cu_seqlens), _p(out),
          c_int(out.shape[1]), c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
          c_float(scale), c_int(window), c_int(n_splits), _p(part_o), _p(part_ml), c_void_p(st.data_ptr()), _stream())
    return out


def decode_cluster(q: torch.Tensor, q_ld: int, kcache: torch.Tensor, vcache: torch.Tensor, page_table, seq_slot, seq_len,
                   cu_seqlens, out: torch.Tensor, *, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int,
                   page_size: int, scale: float, window: int, n_splits: int, part_o=None, part_ml=None) -> torch.Tensor:
    """The same kernel with the 2..8 splits of a (sequence, kv head) as one thread-block cluster that merges
    its partial results through distributed shared memory: no scratch (`part_o`, `part_ml` are not
    used), one kernel."""
    _need_cuda(q, kcache, vcache, page_table, seq_slot, seq_len, cu_seqlens, out)
    _need(q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
          and kcache.is_contiguous() and vcache.is_contiguous(), "attention_decode: bf16 contiguous tensors only")
    rows = kcache.shape[0] * kcache.shape[1] * kcache.shape[2]
    mk = _map(1, kcache, rows, head_dim, head_dim)
    mv = _map(1, vcache, rows, head_dim, head_dim)
    st = status_word()
    _call("attention_mma", "ri_attention_decode_tma_cluster", c_void_p(mk.data_ptr()), c_void_p(mv.data_ptr()), _p(q),
          c_int(q_ld), _p(page_table), c_int(page_table.shape[1]), _p(seq_slot), _p(seq_len), _p(cu_seqlens), _p(out),
          c_int(out.shape[1]), c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
          c_float(scale), c_int(window), c_int(n_splits), c_void_p(st.data_ptr()), _stream())
    return out


_capacity: dict = {}


def decode_cluster_capacity(head_dim: int, n_splits: int) -> int:
    """How many clusters of n_splits CTAs of `decode_cluster`'s kernel the current device holds at once
    (asked once per device, head size and split count)."""
    import ctypes
    key = (torch.cuda.current_device(), head_dim, n_splits)
    if key not in _capacity:
        got = c_int(0)
        _call("attention_mma", "ri_attention_decode_tma_cluster_capacity", c_int(head_dim), c_int(n_splits), ctypes.byref(got))
        _capacity[key] = int(got.value)
    return _capacity[key]
