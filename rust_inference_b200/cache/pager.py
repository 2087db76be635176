"""Host-side bookkeeping of the cache: slots, pages and lengths.  Pure Python, no device.

The reference owns one cache per layer for its single sequence, with a length counter,
an append that asserts on overflow and a clear (kv_cache.rs:40-75, :122-124).  Here a
*slot* stands for one sequence of a batch; its keys and values live in pages of
`page_size` positions taken from a shared pool, so that sequences of unequal length
only hold what they use.  A slot is given back when its sequence ends, with all its
pages, and both are handed out again.  Running out of slots, pages or positions is an
exception raised before anything is launched, never a device fault.
"""
from __future__ import annotations


class CacheError(RuntimeError):
    """Misuse of the cache: an unknown or free slot, a slot freed twice."""


class CacheFull(CacheError):
    """No free slot, no free page, or a sequence longer than the cache allows."""


class SlotPager:
    def __init__(self, n_slots: int, n_pages: int, page_size: int, max_seq_len: int):
        if n_slots <= 0 or n_pages <= 0 or page_size <= 0 or max_seq_len <= 0:
            raise ValueError("cache sizes must be positive")
        self.n_slots = n_slots
        self.n_pages = n_pages
        self.page_size = page_size
        self.max_seq_len = max_seq_len
        self.max_pages_per_slot = min(n_pages, -(-max_seq_len // page_size))
        # popped from the end: low numbers go out first
        self._free_slots = list(range(n_slots - 1, -1, -1))
        self._free_pages = list(range(n_pages - 1, -1, -1))
        self._live = [False] * n_slots
        self._length = [0] * n_slots
        self._pages: list[list[int]] = [[] for _ in range(n_slots)]

    # ---- slots ----------------------------------------------------------
    def alloc_slot(self) -> int:
        if not self._free_slots:
            raise CacheFull(f"all {self.n_slots} cache slots are in use")
        s = self._free_slots.pop()
        self._live[s] = True
        self._length[s] = 0
        return s

    def free_slot(self, slot: int) -> None:
        self._check(slot)
        self._free_pages.extend(reversed(self._pages[slot]))
        self._pages[slot] = []
        self._length[slot] = 0
        self._live[slot] = False
        self._free_slots.append(slot)

    def _check(self, slot: int) -> None:
        if not (0 <= slot < self.n_slots):
            raise CacheError(f"slot {slot} does not exist (0..{self.n_slots - 1})")
        if not self._live[slot]:
            raise CacheError(f"slot {slot} is not in use (never allocated, or freed already)")

    # ---- lengths and pages ----------------------------------------------
    def length(self, slot: int) -> int:
        self._check(slot)
        return self._length[slot]

    def pages(self, slot: int) -> list[int]:
        self._check(slot)
        return list(self._pages[slot])

    def pages_needed(self, slot: int, new_length: int) -> int:
        self._check(slot)
        return max(0, -(-new_length // self.page_size) - len(self._pages[slot]))

    def reserve(self, slot: int, new_length: int) -> list[int]:
        """Make room for positions < new_length; returns the pages added (in order)."""
        self._check(slot)
        if new_length > self.max_seq_len:
            raise CacheFull(f"slot {slot}: {new_length} positions exceed max_seq_len {self.max_seq_len}")
        need = self.pages_needed(slot, new_length)
        if need > len(self._free_pages):
            raise CacheFull(
                f"cache is full: slot {slot} needs {need} more pages of {self.page_size} positions, "
                f"{len(self._free_pages)} of {self.n_pages} are free")
        added = [self._free_pages.pop() for _ in range(need)]
        self._pages[slot].extend(added)
        return added

    def reserve_many(self, wants: list[tuple]) -> dict:
        """All-or-nothing `reserve` for several (slot, new_length) pairs."""
        total = 0
        for slot, new_length in wants:
            self._check(slot)
            if new_length > self.max_seq_len:
                raise CacheFull(f"slot {slot}: {new_length} positions exceed max_seq_len {self.max_seq_len}")
            total += self.pages_needed(slot, new_length)
        if total > len(self._free_pages):
            raise CacheFull(
                f"cache is full: the step needs {total} more pages of {self.page_size} positions, "
                f"{len(self._free_pages)} of {self.n_pages} are free")
        return {slot: self.reserve(slot, new_length) for slot, new_length in wants}

    def set_length(self, slot: int, length: int) -> None:
        self._check(slot)
        if length > len(self._pages[slot]) * self.page_size:
            raise CacheError(f"slot {slot}: length {length} exceeds its reserved pages")
        self._length[slot] = length

    # ---- accounting -----------------------------------------------------
    def free_slot_count(self) -> int:
        return len(self._free_slots)

    def free_page_count(self) -> int:
        return len(self._free_pages)

    def live_slots(self) -> list[int]:
        return [s for s in range(self.n_slots) if self._live[s]]

    def audit(self) -> None:
        """Every slot and every page is either free or held, exactly once."""
        held_pages = [p for s in range(self.n_slots) for p in self._pages[s]]
        all_pages = sorted(held_pages + self._free_pages)
        if all_pages != list(range(self.n_pages)):
            raise CacheError("page accounting broken: a page is lost or held twice")
        live = [s for s in range(self.n_slots) if self._live[s]]
        if sorted(live + self._free_slots) != list(range(self.n_slots)):
            raise CacheError("slot accounting broken: a slot is lost or held twice")
        for s in range(self.n_slots):
            if not self._live[s] and (self._pages[s] or self._length[s]):
                raise CacheError(f"free slot {s} still holds pages or a length")
