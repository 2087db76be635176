"""What one step knows about its batch, and the scratch buffers kernels write into."""
from __future__ import annotations

from dataclasses import dataclass, field
from itertools import chain

import numpy as np
import torch


class Workspace:
    """Named scratch buffers that live across steps, so a step allocates nothing once its
    shapes have been seen (and their addresses stay put for CUDA graphs).  A buffer is
    reused by every layer that asks for the same name: the stream orders the uses."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._flat: dict = {}

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        flat = self._flat.get(key)
        if flat is None or flat.numel() < n:
            flat = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._flat[key] = flat
        return flat[:n].view(*shape)

    def get_zeroed(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        """A buffer that holds zeros whenever it is handed out: it is zero-filled when made, and
        whoever uses it must leave it zeroed again (the kernel that consumes an accumulator puts
        the zeros back).  `rezero` restores that after a step that did not finish."""
        n = 1
        for s in shape:
            n *= int(s)
        key = ("zeroed:" + name, dtype)
        flat = self._flat.get(key)
        if flat is None or flat.numel() < n:
            flat = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._flat[key] = flat
        return flat[:n].view(*shape)

    def rezero(self) -> None:
        for (name, _), flat in self._flat.items():
            if isinstance(name, str) and name.startswith("zeroed:"):
                flat.zero_()

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._flat.values())


@dataclass
class StepContext:
    """A packed batch: T tokens of B sequences, sequence after sequence, no padding.

    token_ids[t], token_pos[t] (absolute position in its sequence), token_seq[t] (which of
    the B sequences), seq_slot[b] (cache slot), seq_start[b] (cached positions before the
    step), seq_len[b] (after it), cu_seqlens[b] (first token of sequence b; [B+1]),
    logit_rows[r] (tokens whose logits are wanted).  All int32 on the device."""
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor
    token_pos: torch.Tensor
    token_seq: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_len: torch.Tensor
    cu_seqlens: torch.Tensor
    logit_rows: torch.Tensor
    n_logit_rows: int
    max_new: int                  # most tokens any sequence brings in this step
    max_len: int                  # longest sequence after the step
    all_single: bool              # every sequence brings exactly one token (a decode step)
    page_table: torch.Tensor
    page_size: int
    dtype: torch.dtype
    device: torch.device
    workspace: Workspace
    extras: dict = field(default_factory=dict)
    # host copies of the per-sequence arrays (None inside a captured graph, whose arrays change
    # between replays): for parts that are not graph_safe
    host_slots: list | None = None
    host_starts: list | None = None
    host_counts: list | None = None

    def buffer(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype)

    def zeroed_buffer(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.get_zeroed(name, shape, dtype)


_pack = None


def _packer():
    global _pack
    if _pack is None:
        from ctypes import c_int, c_longlong, c_void_p
        from ..kernels import build
        fn = build.load("host_runtime").ri_pack_step
        fn.restype = c_longlong
        fn.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p]
        _pack = fn
    return _pack


def pack_step(starts: list, tokens: list, wants: list) -> tuple:
    """Host side of a step: flatten B token lists into the int32 arrays of StepContext (the native
    host runtime lays them out, `csrc/host_runtime.cpp`).

    starts[b]  positions already cached for sequence b
    tokens[b]  its new tokens
    wants[b]   indices into tokens[b] whose logits are wanted
    Returns (meta: np.int32 array, layout: dict name -> (offset, count), scalars: dict)."""
    n_seqs = len(tokens)
    counts = np.fromiter((len(t) for t in tokens), dtype=np.int32, count=n_seqs)
    want_counts = np.fromiter((len(w) for w in wants), dtype=np.int32, count=n_seqs)
    n_tokens, n_rows = int(counts.sum()), int(want_counts.sum())
    flat = np.fromiter(chain.from_iterable(tokens), dtype=np.int32, count=n_tokens) if n_tokens else np.zeros(1, np.int32)
    flat_wants = np.fromiter(chain.from_iterable(wants), dtype=np.int32, count=n_rows) if n_rows else np.zeros(1, np.int32)
    start_arr = np.asarray(starts, dtype=np.int32).reshape(n_seqs)
    sizes = [("token_ids", n_tokens), ("token_pos", n_tokens), ("token_seq", n_tokens),
             ("seq_slot", n_seqs), ("seq_start", n_seqs), ("seq_len", n_seqs),
             ("cu_seqlens", n_seqs + 1), ("logit_rows", n_rows)]
    layout, off = {}, 0
    for name, cnt in sizes:
        layout[name] = (off, cnt)
        off += cnt
    meta = np.zeros(max(off, 1), dtype=np.int32)
    sc = np.zeros(3, dtype=np.int32)
    rc = _packer()(n_seqs, start_arr.ctypes.data, counts.ctypes.data, flat.ctypes.data, None, want_counts.ctypes.data,
                   flat_wants.ctypes.data, meta.ctypes.data, meta.size, sc.ctypes.data)
    if rc < 0:
        from ..kernels import build
        raise ValueError(build.load("host_runtime").ri_last_error().decode())
    scalars = {
        "n_tokens": n_tokens, "n_seqs": n_seqs, "n_logit_rows": n_rows,
        "max_new": int(sc[0]), "max_len": int(sc[1]), "all_single": bool(sc[2]),
    }
    return meta, layout, scalars
