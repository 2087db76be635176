"""Python face of the tcgen05 + TMA contraction kernel (bf16 operands, float32 accumulate)."""
from __future__ import annotations

import functools
from ctypes import byref, c_int, c_longlong, c_void_p

import torch

from . import build, ops
from .ops import KernelError, _call, _need, _need_cuda, _p, _stream

_status = None     # host-visible word a kernel writes when one of its bounded waits ran out
_x_maps: dict = {}  # tensor maps of activation buffers, by (pointer, rows, K, token tile)

STATUS_TEXT = {
    1: "the TMA producer waited too long for a free stage",
    2: "the MMA issuer waited too long for a TMA load",
    3: "the epilogue waited too long for the accumulator",
    4: "a TMA load did not land before the CTA had to leave",
    11: "attention: the TMA producer waited too long for a free page buffer",
    12: "attention: the MMA issuer waited too long for a page or for the softmax",
    13: "attention: the softmax waited too long for scores or for the previous product",
    14: "attention: a TMA load did not land before the CTA had to leave",
    15: "attention: the shared-memory window is not aligned as the tight layout needs",
    21: "decode attention: the TMA producer waited too long for a free stage",
    22: "decode attention: a compute warp waited too long for a page",
    24: "decode attention: a TMA load did not land before the CTA had to leave",
}


def status_word() -> torch.Tensor:
    global _status
    if _status is None:
        _status = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _status


def check_status() -> None:
    """Raise if any tensor-core kernel since the last check gave up on a wait.  Call after a
    synchronisation point (the word lives in pinned host memory the device writes to)."""
    if _status is not None and int(_status[0]) != 0:
        code = int(_status[0])
        _status[0] = 0
        raise KernelError(f"a tensor-core kernel gave up: {STATUS_TEXT.get(code, f'code {code}')}")


def wait_probe(limit: int = 2000, code: int = 2, arrive_first: bool = False) -> None:
    """Run the kernels' bounded wait (`mbar_wait`) on a barrier that nothing arrives at, with a limit
    of `limit` polls: it runs out within microseconds, stores `code` in the status word as a kernel
    that gave up would, and returns.  After a synchronisation `check_status()` raises that code's
    text.  With arrive_first the barrier is complete before the wait, which then succeeds."""
    st = status_word()
    _call("wait_probe", "ri_wait_probe", c_int(limit), c_int(code), c_int(1 if arrive_first else 0),
          c_void_p(st.data_ptr()), _stream())


def supports(x: torch.Tensor, w) -> bool:
    """The kernel's alignment rule: bf16, K a multiple of 8 (16-byte rows for TMA)."""
    return x.dtype == torch.bfloat16 and w.t.dtype == torch.bfloat16 and w.k % 8 == 0 and w.k >= 8


@functools.lru_cache(maxsize=4096)
def plan(n_tok: int, n_feat: int, k: int, mode: int) -> tuple:
    """(token tile, K split) of a product, as the kernel library cuts it: the step rounded up to 16
    up to 128 tokens (with the residual epilogue split over about two CTAs per SM); beyond, 128
    tokens for the SiLU-gate projection (token-major kernel) and for the others the width of
    128..256 and the split that leave the shortest run in the persistent grid."""
    lib = build.load("gemm_tcgen05")
    tile, split = c_int(0), c_int(0)
    lib.ri_gemm_tcgen05_plan(c_int(n_tok), c_int(n_feat), c_int(k), c_int(mode), byref(tile), byref(split))
    return tile.value, split.value


def set_pairs(min_tokens: int = 512, always: bool = False) -> None:
    """Steps of at least `min_tokens` tokens may run on pairs of SMs (tcgen05 cta_group::2; 0: never);
    with `always` they do, whatever their tiles make of the grid.  For comparisons and tests."""
    build.load("gemm_tcgen05").ri_gemm_tcgen05_set_pairs(c_int(min_tokens), c_int(1 if always else 0))
    plan.cache_clear()
    _x_maps.clear()


def token_tile(n_tok: int, n_feat: int, k: int, mode: int) -> int:
    return plan(n_tok, n_feat, k, mode)[0]


def pick_split(n_tok: int, n_feat: int, k: int) -> int:
    """K splits of the residual epilogue for a product of this size."""
    return plan(n_tok, n_feat, k, ops.EPI_RESIDUAL)[1]


def _encode(t: torch.Tensor, rows: int, k: int, box_rows: int) -> torch.Tensor:
    m = torch.empty(128, dtype=torch.uint8)           # CPU allocations are 64-byte aligned
    _call("gemm_tcgen05", "ri_gemm_tcgen05_encode", c_void_p(m.data_ptr()), _p(t), c_longlong(rows),
          c_longlong(k), c_int(box_rows))
    ops._launches -= 1                                # encoding a map launches nothing
    return m


def weight_map(w) -> torch.Tensor:
    if w.tc is None:
        w.tc = _encode(w.t, w.n, w.k, 128)
    return w.tc


def _x_map(x: torch.Tensor, tn: int) -> torch.Tensor:
    key = (x.data_ptr(), x.shape[0], x.shape[1], tn)
    m = _x_maps.get(key)
    if m is None:
        if len(_x_maps) > 8192:
            _x_maps.clear()
        m = _x_maps[key] = _encode(x, x.shape[0], x.shape[1], tn)
    return m


def gemm(x: torch.Tensor, w, out: torch.Tensor, mode: int, ctx=None, bias=None, w2=None, split_k: int | None = None):
    _need_cuda(x, w.t, out, bias)
    m, k = x.shape
    n = w.n
    _need(w.k == k and x.dtype == torch.bfloat16 and w.t.dtype == torch.bfloat16 and x.is_contiguous()
          and out.is_contiguous() and out.shape == (m, n), "gemm_tcgen05: bad shapes or dtypes")
    want_out = torch.float32 if mode in (ops.EPI_STORE_F32, ops.EPI_RESIDUAL) else torch.bfloat16
    _need(out.dtype == want_out, f"gemm_tcgen05: epilogue {mode} writes {want_out}, out is {out.dtype}")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm_tcgen05: bias must be float32 [N]")
    map_w2 = None
    if w2 is not None:
        _need((w2.n, w2.k) == (n, k) and w2.t.dtype == torch.bfloat16, "gemm_tcgen05: second matrix")
        map_w2 = weight_map(w2)
    if m == 0:
        return out
    tile, planned = plan(m, n, k, mode)
    if split_k is None:
        split_k = planned
    map_x = _x_map(x, tile)
    st = status_word()
    _call("gemm_tcgen05", "ri_gemm_tcgen05", c_void_p(map_x.data_ptr()), c_void_p(weight_map(w).data_ptr()),
          c_void_p(map_w2.data_ptr() if map_w2 is not None else 0), _p(bias), _p(out), c_int(mode), c_int(m),
          c_int(n), c_int(k), c_int(split_k), c_void_p(st.data_ptr()), _stream())
    return out
