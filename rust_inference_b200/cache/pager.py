"""Host-side bookkeeping of the cache: slots, pages and lengths.  No device.

The reference owns one cache per layer for its single sequence, with a length counter,
an append that asserts on overflow and a clear (kv_cache.rs:40-75, :122-124).  Here a
*slot* stands for one sequence of a batch; its keys and values live in pages of
`page_size` positions taken from a shared pool, so that sequences of unequal length
only hold what they use.  A slot is given back when its sequence ends, with all its
pages, and both are handed out again.  Running out of slots, pages or positions is an
exception raised before anything is launched, never a device fault.

The books themselves are kept by the native host runtime (`csrc/host_runtime.cpp`);
this class is its face: it owns the handle, passes arrays and turns error codes into
exceptions.
"""
from __future__ import annotations

from ctypes import c_int, c_void_p

import numpy as np

_FULL, _NO_SUCH_SLOT, _NOT_LIVE, _TOO_LONG, _BAD_LENGTH = -1, -2, -3, -4, -5


class CacheError(RuntimeError):
    """Misuse of the cache: an unknown or free slot, a slot freed twice."""


class CacheFull(CacheError):
    """No free slot, no free page, or a sequence longer than the cache allows."""


_lib = None


def _runtime():
    global _lib
    if _lib is None:
        from ..kernels import build
        lib = build.load("host_runtime")
        lib.ri_pager_create.restype = c_void_p
        lib.ri_pager_create.argtypes = [c_int, c_int, c_int, c_int]
        lib.ri_pager_destroy.restype = None
        lib.ri_pager_destroy.argtypes = [c_void_p]
        lib.ri_pager_prefer_high_pages.restype = None
        lib.ri_pager_prefer_high_pages.argtypes = [c_void_p]
        for name, args in (("alloc_slot", []), ("free_slot", [c_int]), ("length", [c_int]), ("page_count", [c_int]),
                           ("pages", [c_int, c_void_p, c_int]), ("pages_needed", [c_int, c_int]),
                           ("reserve_many", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int]),
                           ("set_length", [c_int, c_int]), ("free_slot_count", []), ("free_page_count", []),
                           ("live_slots", [c_void_p]), ("audit", []), ("lengths", [c_int, c_void_p, c_void_p]),
                           ("advance", [c_int, c_void_p, c_void_p])):
            fn = getattr(lib, "ri_pager_" + name)
            fn.restype = c_int
            fn.argtypes = [c_void_p] + args
        _lib = lib
    return _lib


class SlotPager:
    def __init__(self, n_slots: int, n_pages: int, page_size: int, max_seq_len: int):
        if n_slots <= 0 or n_pages <= 0 or page_size <= 0 or max_seq_len <= 0:
            raise ValueError("cache sizes must be positive")
        self.n_slots = n_slots
        self.n_pages = n_pages
        self.page_size = page_size
        self.max_seq_len = max_seq_len
        self.max_pages_per_slot = min(n_pages, -(-max_seq_len // page_size))
        self._rt = _runtime()
        self._h = c_void_p(self._rt.ri_pager_create(n_slots, n_pages, page_size, max_seq_len))
        if not self._h:
            raise ValueError(self._rt.ri_last_error().decode())
        self._scratch = np.zeros(max(n_slots, self.max_pages_per_slot, 64), dtype=np.int32)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                self._rt.ri_pager_destroy(h)
            except Exception:          # the interpreter is shutting down and the library is gone
                pass

    def _raise(self, code: int):
        msg = self._rt.ri_last_error().decode()
        raise (CacheFull if code in (_FULL, _TOO_LONG) else CacheError)(msg)

    def _call(self, name: str, *args) -> int:
        rc = getattr(self._rt, "ri_pager_" + name)(self._h, *args)
        if rc < 0:
            self._raise(rc)
        return rc

    # ---- slots ----------------------------------------------------------
    def alloc_slot(self) -> int:
        return self._call("alloc_slot")

    def free_slot(self, slot: int) -> None:
        self._call("free_slot", int(slot))

    # ---- lengths and pages ----------------------------------------------
    def length(self, slot: int) -> int:
        return self._call("length", int(slot))

    def lengths(self, slots: list) -> list[int]:
        a = np.asarray(slots, dtype=np.int32)
        out = np.empty(max(a.size, 1), dtype=np.int32)
        self._call("lengths", a.size, a.ctypes.data, out.ctypes.data)
        return out[:a.size].tolist()

    def advance(self, slots: list, counts: list) -> None:
        """Every slot's length moves on by its count (the end of a step); all or none."""
        a, c = np.asarray(slots, dtype=np.int32), np.asarray(counts, dtype=np.int32)
        if a.size != c.size:
            raise ValueError("advance: one count per slot")
        self._call("advance", a.size, a.ctypes.data, c.ctypes.data)

    def page_count(self, slot: int) -> int:
        return self._call("page_count", int(slot))

    def pages(self, slot: int) -> list[int]:
        buf = self._scratch
        n = self._call("pages", int(slot), buf.ctypes.data, buf.size)
        return buf[:n].tolist()

    def pages_needed(self, slot: int, new_length: int) -> int:
        return self._call("pages_needed", int(slot), int(new_length))

    def reserve(self, slot: int, new_length: int) -> list[int]:
        """Make room for positions < new_length; returns the pages added (in order)."""
        return self.reserve_many([(slot, new_length)])[slot]

    def reserve_many(self, wants: list[tuple]) -> dict:
        """All-or-nothing `reserve` for several (slot, new_length) pairs: slot -> pages added."""
        n = len(wants)
        pairs = np.asarray(wants, dtype=np.int64).reshape(n, 2)
        if n and (np.abs(pairs) > 0x7fffffff).any():
            raise CacheFull("a length beyond the index range")
        slots = np.ascontiguousarray(pairs[:, 0], dtype=np.int32)
        lengths = np.ascontiguousarray(pairs[:, 1], dtype=np.int32)
        counts = np.zeros(max(n, 1), dtype=np.int32)
        cap = int(sum(max(0, -(-int(length) // self.page_size)) for length in lengths)) + 1
        added = np.zeros(cap, dtype=np.int32)
        self._call("reserve_many", n, slots.ctypes.data, lengths.ctypes.data, counts.ctypes.data, added.ctypes.data, cap)
        out: dict = {}
        off = 0
        for i in range(n):
            c = int(counts[i])
            out.setdefault(int(slots[i]), []).extend(added[off:off + c].tolist())
            off += c
        return out

    def set_length(self, slot: int, length: int) -> None:
        self._call("set_length", int(slot), int(length))

    # ---- accounting -----------------------------------------------------
    def free_slot_count(self) -> int:
        return self._call("free_slot_count")

    def free_page_count(self) -> int:
        return self._call("free_page_count")

    def live_slots(self) -> list[int]:
        buf = self._scratch
        n = self._call("live_slots", buf.ctypes.data)
        return buf[:n].tolist()

    def prefer_high_pages(self) -> None:
        """Hand out the highest page numbers first from now on (for tests that want a sequence at
        the far end of the pool)."""
        self._rt.ri_pager_prefer_high_pages(self._h)

    def audit(self) -> None:
        """Every slot and every page is either free or held, exactly once."""
        if self._rt.ri_pager_audit(self._h) != 0:
            raise CacheError(self._rt.ri_last_error().decode())
