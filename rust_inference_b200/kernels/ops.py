"""Python faces of the CUDA kernels: they check the tensors they are given, pass raw
pointers and the current CUDA stream to the C ABI, and raise on any error.

There is no other implementation behind them.  A tensor that is not on a CUDA device,
a missing compiler or a library that does not load is an error, never a detour.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_float, c_void_p, c_longlong, c_ulonglong

import torch

from .build import load

RI_F32, RI_BF16 = 0, 1
_DTYPE_CODE = {torch.float32: RI_F32, torch.bfloat16: RI_BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _p(t) -> c_void_p:
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel called with a tensor that is not on a CUDA device; "
                              "this library has no CPU path")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


_launches = 0


def launch_count() -> int:
    """How many kernel entry points have been called (each launches one kernel)."""
    return _launches


_limits = None          # checked build: (vocabulary, slots, pages) for libraries still to be loaded
_limited: set = set()   # libraries that have them


def _call(module: str, fn: str, *args) -> None:
    global _launches
    lib = load(module)
    if _limits is not None and module not in _limited:
        _apply_limits(module, lib)
    rc = getattr(lib, fn)(*args)
    if rc != 0:
        raise KernelError(f"{fn}: {lib.ri_last_error().decode()}")
    _launches += 1


# ----------------------------------------------------------------------------
# The checked build (RI_B200_CHECK_BOUNDS=1)
# ----------------------------------------------------------------------------
BOUND_CHECKS = {1: "a token id outside the vocabulary", 2: "a cache slot that does not exist",
                3: "a position beyond a sequence's page table", 4: "a page that does not exist"}


def checked_build() -> bool:
    from . import build
    return build.CHECKED


def _apply_limits(module: str, lib) -> None:
    from . import build
    if build.MODULES[module].endswith(".cu"):
        if lib.ri_bounds_set_limits(c_int(_limits[0]), c_int(_limits[1]), c_int(_limits[2])) != 0:
            raise KernelError(f"{module}: {lib.ri_last_error().decode()}")
    _limited.add(module)


def bounds_set_limits(vocab: int, slots: int, pages: int) -> None:
    """Checked build only: the limits that kernels are not given as arguments (0: not checked), for
    every CUDA library loaded so far and, at its first call, every one loaded later."""
    global _limits
    from . import build
    _limits = (int(vocab), int(slots), int(pages))
    _limited.clear()
    for module in build.loaded_cuda_modules():
        _apply_limits(module, load(module))


def bounds_report() -> list:
    """Checked build only: what the kernels recorded since the last call, per library:
    (library, what was outside, the index, its limit, how many indices were outside).  Reads the
    records back (synchronises the device) and clears them."""
    from . import build
    out = []
    for module in build.loaded_cuda_modules():
        lib = load(module)
        rec = (c_int * 4)()
        if lib.ri_bounds_report(rec) != 0:
            raise KernelError(f"{module}: {lib.ri_last_error().decode()}")
        if rec[3]:
            out.append((module, BOUND_CHECKS.get(rec[0], f"check {rec[0]}"), rec[1], rec[2], rec[3]))
    return out


# ----------------------------------------------------------------------------
# The timeline build (RI_B200_TIMELINE=1)
# ----------------------------------------------------------------------------
TIMELINE_PHASES = 6


def timeline_build() -> bool:
    from . import build
    return build.TIMELINE


def timeline_read(strict: bool = True) -> list:
    """Timeline build only: one record per kernel launched since the last call, in the order the kernels
    came onto the device: {"module", "entry_ns", "entry_line", "wait_ns", "wait_line", "phases_ns"} with
    the device-wide timer's values (0: that mark was not passed) and the source lines of the kernel's
    `let_next_kernel_start()` and `wait_for_previous_kernels()`.  Synchronises the device and clears
    the records.  `strict`: raise when launches fell on the same record (thousands since the last read)."""
    import ctypes
    from . import build
    words = 5 + TIMELINE_PHASES
    cap = 4096
    out = []
    for module in build.loaded_cuda_modules():
        lib = load(module)
        buf = (ctypes.c_ulonglong * (cap * words))()
        n = lib.ri_timeline_read(buf, c_int(cap))
        if n < 0:
            raise KernelError(f"{module}: {lib.ri_last_error().decode()}")
        found = 0
        for i in range(cap):
            if buf[i * words]:
                r = buf[i * words:(i + 1) * words]
                out.append({"module": module, "entry_ns": r[0], "entry_line": r[1], "wait_ns": r[2], "wait_line": r[3],
                            "grid": r[4] - 1, "phases_ns": list(r[5:])})
                found += 1
        if strict and found != n:
            raise KernelError(f"{module}: {n} launches since the last read but {found} records: launches fell on "
                              f"the same record (the timeline keeps {cap})")
    out.sort(key=lambda r: r["entry_ns"])
    return out


# ----------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] widened to float32.  ids: int32 [T]; out: float32 [T, H]."""
    _need_cuda(table, ids, out)
    n, hidden = out.shape
    _need(ids.dtype == torch.int32 and ids.numel() == n, "embed_gather: ids must be int32 [T]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
          and table.shape[1] == hidden, "embed_gather: bad out/table")
    _call("elementwise", "ri_embed_gather", _p(table), c_int(dtype_code(table.dtype)), _p(ids), _p(out),
          c_int(n), c_int(hidden), _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, :] = rmsnorm(x[rows[r] or r, :]) * weight.  x, weight float32; out float32 or bfloat16."""
    _need_cuda(x, weight, out, rows)
    n_rows, n = out.shape
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32, "rmsnorm: x and weight must be float32")
    _need(x.is_contiguous() and out.is_contiguous() and x.shape[-1] == n and weight.numel() == n,
          "rmsnorm: bad shapes")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() == n_rows, "rmsnorm: rows must be int32 [R]")
    else:
        _need(x.shape[0] >= n_rows, "rmsnorm: x has fewer rows than out")
    _call("elementwise", "ri_rmsnorm", _p(x), _p(weight), _p(rows), _p(out), c_int(dtype_code(out.dtype)),
          c_int(n_rows), c_int(n), c_float(eps), _stream())
    return out


def rope_cache_write(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, token_pos, token_seq,
                     seq_slot, page_table: torch.Tensor, kcache, vcache, *, n_heads: int,
                     n_kv_heads: int, head_dim: int, page_size: int, style: int, write_kv: bool) -> None:
    """Rotate q (in place) and k by the table rows of each token's position; store rotated k and v
    at the token's cache position.  kcache/vcache: one layer, [pages, kv heads, page_size, head_dim]."""
    _need_cuda(qkv, cos, sin, token_pos, token_seq, seq_slot, page_table, kcache, vcache)
    n = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim,
          "rope_cache_write: qkv must be [T, (heads + 2 kv heads) * head_dim]")
    _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape[1] == head_dim // 2,
          "rope_cache_write: tables must be float32 [positions, head_dim/2]")
    if write_kv:
        _need(kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype and kcache.is_contiguous()
              and vcache.is_contiguous(), "rope_cache_write: cache dtype/layout")
        _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "rope_cache_write: cache shape")
    _call("elementwise", "ri_rope_cache_write", _p(qkv), c_int(dtype_code(qkv.dtype)), c_int(qkv.shape[1]),
          _p(cos), _p(sin), _p(token_pos), _p(token_seq), _p(seq_slot), _p(page_table),
          c_int(page_table.shape[1]), _p(kcache), _p(vcache), c_int(n), c_int(n_heads), c_int(n_kv_heads),
          c_int(head_dim), c_int(page_size), c_int(style), c_int(1 if write_kv else 0), _stream())


def rope_cache_write_acc(acc: torch.Tensor, bias, q_out: torch.Tensor, cos, sin, token_pos, token_seq, seq_slot,
                         page_table, kcache, vcache, *, n_heads: int, n_kv_heads: int, head_dim: int,
                         page_size: int, style: int, write_kv: bool) -> None:
    """The rotary + cache-write kernel fed from float32 accumulators acc[T, (heads + 2 kv heads) * head_dim]
    (+ bias): q goes to q_out[T, heads * head_dim], k and v to the cache, and `acc` is zeroed again."""
    _need_cuda(acc, bias, q_out, cos, sin, token_pos, token_seq, seq_slot, page_table, kcache, vcache)
    n = acc.shape[0]
    _need(acc.dtype == torch.float32 and acc.is_contiguous()
          and acc.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim, "rope_cache_write_acc: accumulator shape")
    _need(q_out.is_contiguous() and q_out.shape == (n, n_heads * head_dim), "rope_cache_write_acc: q_out shape")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == acc.shape[1]), "rope_cache_write_acc: bias")
    if write_kv:
        _need(kcache.dtype == q_out.dtype and vcache.dtype == q_out.dtype
              and tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "rope_cache_write_acc: cache")
    _call("elementwise", "ri_rope_cache_write_acc", _p(acc), c_int(acc.shape[1]), _p(bias), _p(q_out),
          c_int(dtype_code(q_out.dtype)), _p(cos), _p(sin), _p(token_pos), _p(token_seq), _p(seq_slot),
          _p(page_table), c_int(page_table.shape[1]), _p(kcache), _p(vcache), c_int(n), c_int(n_heads),
          c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_int(style), c_int(1 if write_kv else 0), _stream())


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need_cuda(gate_up, out)
    n, inter = out.shape
    _need(gate_up.shape == (n, 2 * inter) and gate_up.dtype == out.dtype and gate_up.is_contiguous()
          and out.is_contiguous(), "silu_mul: bad shapes")
    _call("elementwise", "ri_silu_mul", _p(gate_up), _p(out), c_int(dtype_code(out.dtype)), c_int(n),
          c_int(inter), _stream())
    return out


# epilogues of the contractions
EPI_STORE, EPI_STORE_F32, EPI_RESIDUAL, EPI_SILU_MUL = 0, 1, 2, 3


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, *,
              bias: torch.Tensor | None = None, w2: torch.Tensor | None = None) -> torch.Tensor:
    """out = x @ w.T with the chosen epilogue, on the FFMA pipe (float32 accumulate)."""
    _need_cuda(x, w, out, bias, w2)
    m, k = x.shape
    n = w.shape[0]
    _need(w.shape[1] == k and x.dtype == w.dtype and x.is_contiguous() and w.is_contiguous()
          and out.is_contiguous() and out.shape == (m, n), "gemm: bad shapes")
    want_out = torch.float32 if mode in (EPI_STORE_F32, EPI_RESIDUAL) else x.dtype
    _need(out.dtype == want_out, f"gemm: epilogue {mode} writes {want_out}, out is {out.dtype}")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm: bias must be float32 [N]")
    if w2 is not None:
        _need(w2.shape == w.shape and w2.dtype == w.dtype and w2.is_contiguous(), "gemm: second matrix")
    _call("gemm_simt", "ri_gemm_simt", _p(x), _p(w), _p(w2), _p(bias), _p(out), c_int(dtype_code(x.dtype)),
          c_int(mode), c_int(m), c_int(n), c_int(k), _stream())
    return out


def attention_generic(q: torch.Tensor, q_ld: int, kcache, vcache, page_table, token_pos, token_seq,
                      seq_slot, out: torch.Tensor, *, n_tokens: int, n_heads: int, n_kv_heads: int,
                      head_dim: int, page_size: int, scale: float, window: int = 0) -> torch.Tensor:
    """Attention of every given token over its slot's cached keys 0..position (any sizes)."""
    _need_cuda(q, kcache, vcache, page_table, token_pos, token_seq, seq_slot, out)
    _need(q.dtype == kcache.dtype == vcache.dtype == out.dtype, "attention: dtypes differ")
    _need(out.is_contiguous() and out.shape == (n_tokens, n_heads * head_dim), "attention: out shape")
    rows = kcache.shape[0] * kcache.shape[1] * kcache.shape[2]
    _call("attention_generic", "ri_attention_generic", _p(q), c_int(q_ld), _p(kcache), _p(vcache),
          _p(page_table), c_int(page_table.shape[1]), _p(token_pos), _p(token_seq), _p(seq_slot), _p(out),
          c_int(out.shape[1]), c_int(dtype_code(q.dtype)), c_int(n_tokens), c_int(n_heads),
          c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_longlong(rows), c_float(scale),
          c_int(window), _stream())
    return out


def sample(logits: torch.Tensor, out: torch.Tensor, *, temperature: float, top_k: int = 0, top_p: float = 1.0,
           penalty: float = 1.0, recent: torch.Tensor | None = None, recent_count: torch.Tensor | None = None,
           seed: int = 0, row_stream: torch.Tensor | None = None,
           row_counter: torch.Tensor | None = None, counter_offset: int = 0,
           mirror: torch.Tensor | None = None, newest: torch.Tensor | None = None,
           seed_dev: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V] (overwritten).  out: int32 [R].  `mirror`: a
    pinned int32 host tensor [R] that receives the tokens as well (the kernel writes it directly).
    `newest`: int32 [R] on the device, one more recent id per row for the repetition penalty.
    `seed_dev`: int64 [1] on the device, a seed that takes the place of `seed` (read when the kernel runs)."""
    _need(seed_dev is None or (seed_dev.is_cuda and seed_dev.dtype == torch.int64 and seed_dev.numel() >= 1),
          "sample: seed_dev must be int64 [1] on the device")
    _need_cuda(logits, out, recent, recent_count, row_stream, row_counter, newest)
    _need(newest is None or (newest.dtype == torch.int32 and newest.is_contiguous() and newest.numel() >= logits.shape[0]),
          "sample: newest must be int32 [R]")
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits must be contiguous float32")
    _need(out.dtype == torch.int32 and out.numel() >= rows, "sample: out must be int32 [R]")
    for t in (recent, recent_count, row_stream, row_counter):
        _need(t is None or (t.dtype == torch.int32 and t.is_contiguous()), "sample: index tensors must be int32")
    _need((recent is None) == (recent_count is None), "sample: recent and recent_count go together")
    if mirror is not None:
        _need(mirror.device.type == "cpu" and mirror.is_pinned() and mirror.dtype == torch.int32
              and mirror.is_contiguous() and mirror.numel() >= rows, "sample: mirror must be pinned int32 [R]")
    _call("sampling", "ri_sample", _p(logits), c_int(rows), c_int(vocab), _p(out), c_float(temperature),
          c_int(top_k), c_float(top_p), c_float(penalty), _p(recent),
          c_int(recent.shape[1] if recent is not None else 0), _p(recent_count),
          c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _p(row_stream), _p(row_counter), c_int(counter_offset),
          c_void_p(mirror.data_ptr() if mirror is not None else 0), _p(newest), _p(seed_dev), _stream())
    return out


def cast(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """src (float32 or bfloat16, contiguous, on the device) in the other of the two precisions."""
    _need_cuda(src)
    _need(src.is_contiguous(), "cast: contiguous tensors only")
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    _call("elementwise", "ri_cast", _p(src), c_int(dtype_code(src.dtype)), _p(out), c_int(dtype_code(dtype)),
          c_longlong(src.numel()), _stream())
    return out


def fill_normal(out: torch.Tensor, key: int, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
    """out[i] = mean + std * z_i with z_i a standard normal number that depends on (key, i) only
    (`sampling.rng.normal` restates it on the host).  out: float32 or bfloat16, contiguous, on the device."""
    _need_cuda(out)
    _need(out.is_contiguous(), "fill_normal: contiguous tensors only")
    _call("elementwise", "ri_fill_normal", _p(out), c_int(dtype_code(out.dtype)), c_longlong(out.numel()),
          c_ulonglong(key & 0xFFFFFFFFFFFFFFFF), c_float(mean), c_float(std), _stream())
    return out


def advance_decode(token_pos: torch.Tensor, seq_start: torch.Tensor, seq_len: torch.Tensor, token_ids: torch.Tensor,
                   *, draw_counter: torch.Tensor | None = None, turn: torch.Tensor | None = None,
                   host_ring: torch.Tensor | None = None, log_ring: torch.Tensor | None = None) -> None:
    """The end of a decode step: positions, starts and lengths (int32 [n] each) grow by one in
    place.  Optionally the sampler's draw counters grow by one, and the step's tokens are copied
    into slot (turn % slots) of `host_ring` (pinned int32 [slots, n]) and of `log_ring` (device int32
    [slots, n]); `turn` (device int32 [1]) then grows by one."""
    n = token_pos.numel()
    _need_cuda(token_pos, seq_start, seq_len, token_ids, draw_counter, turn, log_ring)
    for t in (token_pos, seq_start, seq_len, token_ids, draw_counter, turn, log_ring):
        _need(t is None or (t.dtype == torch.int32 and t.is_contiguous()), "advance_decode: arrays must be int32")
    _need(seq_start.numel() == n and seq_len.numel() == n and token_ids.numel() >= n
          and (draw_counter is None or draw_counter.numel() >= n), "advance_decode: one entry per sequence")
    if host_ring is not None:
        _need(host_ring.device.type == "cpu" and host_ring.is_pinned() and host_ring.dtype == torch.int32
              and host_ring.is_contiguous() and host_ring.ndim == 2 and host_ring.shape[1] == n,
              "advance_decode: host_ring must be pinned int32 [slots, n]")
    if log_ring is not None:
        _need(log_ring.ndim == 2 and log_ring.shape[1] == n, "advance_decode: log_ring must be int32 [slots, n]")
    _need((host_ring is None and log_ring is None) or turn is not None, "advance_decode: rings need the turn counter")
    _call("elementwise", "ri_advance_decode", _p(token_pos), _p(seq_start), _p(seq_len), c_int(n), _p(token_ids),
          _p(draw_counter), _p(turn), c_void_p(host_ring.data_ptr() if host_ring is not None else 0),
          c_int(host_ring.shape[0] if host_ring is not None else 0), _p(log_ring),
          c_int(log_ring.shape[0] if log_ring is not None else 0), _stream())


def sample_cluster_min_vocab(vocab: int) -> None:
    """Rows of at least `vocab` entries are sampled by a cluster of thread blocks where the options
    allow it (0: never; the library's default is 32,768).  For comparisons and tests."""
    load("sampling").ri_sample_set_cluster_min_vocab(c_int(vocab))


def sample_cluster_any_rows(on: bool) -> None:
    """Whether such rows are sampled by clusters however many rows a call brings (the library's default:
    only while the clusters are few enough to run together; more rows take a block each).  For
    comparisons and tests."""
    load("sampling").ri_sample_set_cluster_any_rows(c_int(1 if on else 0))


def attention_mma_supports(head_dim: int, page_size: int, n_heads: int, n_kv_heads: int, decode: bool) -> bool:
    lib = load("attention_mma")
    return bool(lib.ri_attention_mma_supports(c_int(head_dim), c_int(page_size), c_int(n_heads),
                                              c_int(n_kv_heads), c_int(1 if decode else 0)))


def attention_decode(q: torch.Tensor, q_ld: int, kcache, vcache, page_table, seq_slot, seq_len, cu_seqlens,
                     out: torch.Tensor, *, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int,
                     page_size: int, scale: float, window: int, n_splits: int, part_o=None, part_ml=None):
    """bf16 attention of one new token per sequence over its slot's keys, split into runs of
    pages; partial results go through the float32 scratch part_o / part_ml when n_splits > 1."""
    _need_cuda(q, kcache, vcache, page_table, seq_slot, seq_len, cu_seqlens, out, part_o, part_ml)
    _need(q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_decode: bf16 only")
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32
              and part_o.numel() >= n_seqs * n_heads * n_splits * head_dim
              and part_ml is not None and part_ml.numel() >= n_seqs * n_heads * n_splits * 2,
              "attention_decode: scratch too small")
    _call("attention_mma", "ri_attention_decode", _p(q), c_int(q_ld), _p(kcache), _p(vcache), _p(page_table),
          c_int(page_table.shape[1]), _p(seq_slot), _p(seq_len), _p(cu_seqlens), _p(out), c_int(out.shape[1]),
          c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_float(scale),
          c_int(window), c_int(n_splits), _p(part_o), _p(part_ml), _stream())
    return out


def attention_prefill(q: torch.Tensor, q_ld: int, kcache, vcache, page_table, seq_slot, seq_start, cu_seqlens,
                      out: torch.Tensor, *, n_seqs: int, max_new: int, n_heads: int, n_kv_heads: int,
                      head_dim: int, page_size: int, scale: float, window: int):
    """bf16 causal attention of every new token of every sequence over its slot's keys."""
    _need_cuda(q, kcache, vcache, page_table, seq_slot, seq_start, cu_seqlens, out)
    _need(q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_prefill: bf16 only")
    _call("attention_mma", "ri_attention_prefill", _p(q), c_int(q_ld), _p(kcache), _p(vcache), _p(page_table),
          c_int(page_table.shape[1]), _p(seq_slot), _p(seq_start), _p(cu_seqlens), _p(out), c_int(out.shape[1]),
          c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
          c_float(scale), c_int(window), _stream())
    return out
