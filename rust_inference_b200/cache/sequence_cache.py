"""The device cache: keys and values for every cache layer, one slot per sequence, and a
fixed-size per-sequence state area beside them.

Layers ask for what they need (`KVRequest`, `StateRequest`); layers with the same needs
form a *group* with storage of its own:

  kv group     K, V: [layers in group, pages, kv heads, page_size, head_dim], in the run
               dtype.  A (page, kv head) is a dense [page_size, head_dim] tile.  Groups are
               keyed by (kv heads, head_dim, window), so layers that keep all keys and
               layers that look at a window do not share storage.
  state group  [layers in group, slots, *shape]: state of fixed size per sequence, zeroed
               when the slot is handed out.  The dense decoder has none; the area exists
               so a mixer with state of its own can be added.

All kv groups share one paging (`SlotPager`): position p of a slot lies in page
`page_table[slot, p // page_size]` at offset `p % page_size`, in every layer.  The
reference's per-layer `[max_seq_len, kv_dim]` pair with one length counter
(kv_cache.rs:25-50) is the one-slot, one-page-per-sequence case of this.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .pager import SlotPager, CacheError, CacheFull  # noqa: F401

PAGE_SIZE = 64


@dataclass(frozen=True)
class KVRequest:
    n_kv_heads: int
    head_dim: int
    window: int | None = None      # None: the layer reads all keys


@dataclass(frozen=True)
class StateRequest:
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class KVLayer:
    k: torch.Tensor                # [pages, kv heads, page_size, head_dim]
    v: torch.Tensor
    request: KVRequest


@dataclass
class StateLayer:
    state: torch.Tensor            # [slots, *shape]
    request: StateRequest


class SequenceCache:
    def __init__(self, requests: list, *, max_tokens: int, max_seq_len: int, dtype: torch.dtype,
                 device, n_slots: int | None = None, page_size: int = PAGE_SIZE):
        """requests[i] is what cache layer i needs (KVRequest, StateRequest or None).
        `max_tokens` is the number of positions all live sequences may hold together, each
        sequence's count rounded up to a whole page."""
        self.device = torch.device(device)
        self.dtype = dtype
        self.page_size = page_size
        n_pages = max(1, -(-max_tokens // page_size))
        max_seq_len = min(max_seq_len, n_pages * page_size)
        if n_slots is None:
            n_slots = min(n_pages, 1024)
        self.pager = SlotPager(n_slots, n_pages, page_size, max_seq_len)
        self.max_seq_len = max_seq_len
        self.n_slots = n_slots
        self.n_pages = n_pages

        self.page_table_host = np.zeros((n_slots, self.pager.max_pages_per_slot), dtype=np.int32)
        self.page_table = torch.zeros((n_slots, self.pager.max_pages_per_slot), dtype=torch.int32,
                                      device=self.device)

        self._stage_bufs = [None] * 4
        self._stage_events = [None] * 4
        self._stage_turn = 0
        self.h2d_bytes = 0             # bytes of page-table entries copied to the device so far

        # group layers by their needs
        self.groups: dict = {}
        self._layers: list = [None] * len(requests)
        members: dict = {}
        for i, req in enumerate(requests):
            if req is not None:
                members.setdefault(req, []).append(i)
        for req, layer_ids in members.items():
            if isinstance(req, KVRequest):
                shape = (len(layer_ids), n_pages, req.n_kv_heads, page_size, req.head_dim)
                k = torch.zeros(shape, dtype=dtype, device=self.device)
                v = torch.zeros(shape, dtype=dtype, device=self.device)
                self.groups[req] = (k, v)
                for j, i in enumerate(layer_ids):
                    self._layers[i] = KVLayer(k[j], v[j], req)
            elif isinstance(req, StateRequest):
                s = torch.zeros((len(layer_ids), n_slots) + tuple(req.shape), dtype=req.dtype,
                                device=self.device)
                self.groups[req] = (s,)
                for j, i in enumerate(layer_ids):
                    self._layers[i] = StateLayer(s[j], req)
            else:
                raise TypeError(f"cache layer {i}: unknown request {req!r}")

    # ---- what the model reads --------------------------------------------
    def layer(self, index: int):
        return self._layers[index]

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for g in self.groups.values() for t in g)

    # ---- slots -------------------------------------------------------------
    def alloc_slot(self) -> int:
        slot = self.pager.alloc_slot()
        for req, tensors in self.groups.items():
            if isinstance(req, StateRequest):
                tensors[0][:, slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        self.pager.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.pager.length(slot)

    def _staging(self, n: int) -> torch.Tensor:
        """A pinned int32 buffer of n entries whose earlier use has been copied out: page-table
        updates go through these, so that publishing them never blocks the host on the stream."""
        i = self._stage_turn
        self._stage_turn = (i + 1) % len(self._stage_bufs)
        if self._stage_events[i] is not None:
            self._stage_events[i].synchronize()
        buf = self._stage_bufs[i]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(256, 2 * n), dtype=torch.int32).pin_memory()
            self._stage_bufs[i] = buf
        return buf

    def reserve(self, wants: list[tuple]) -> None:
        """Make room for (slot, new_length) pairs, all or nothing, and publish the page table
        entries that were added to the device (asynchronously, in stream order)."""
        added = {slot: pages for slot, pages in self.pager.reserve_many(wants).items() if pages}
        if not added:
            return
        total = sum(len(p) for p in added.values())
        self.h2d_bytes += 4 * total
        if self.device.type != "cuda":
            for slot, pages in added.items():
                have = self.pager.page_count(slot)
                self.page_table_host[slot, have - len(pages):have] = pages
                self.page_table[slot, have - len(pages):have] = torch.tensor(pages, dtype=torch.int32)
            return
        buf = self._staging(total)
        off = 0
        for slot, pages in added.items():
            have = self.pager.page_count(slot)
            self.page_table_host[slot, have - len(pages):have] = pages
            buf[off:off + len(pages)] = torch.tensor(pages, dtype=torch.int32)
            self.page_table[slot, have - len(pages):have].copy_(buf[off:off + len(pages)], non_blocking=True)
            off += len(pages)
        ev = torch.cuda.Event()
        ev.record()
        self._stage_events[(self._stage_turn - 1) % len(self._stage_bufs)] = ev

    def commit(self, slot: int, new_length: int) -> None:
        self.pager.set_length(slot, new_length)

    def lengths(self, slots: list) -> list:
        return self.pager.lengths(slots)

    def advance(self, slots: list, counts: list) -> None:
        """The end of a step: every slot's length moves on by the tokens it was given."""
        self.pager.advance(slots, counts)
