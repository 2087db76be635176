"""The sampler: turns a step's logits into one token per sequence, on the device."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .params import SamplerConfig


class Sampler:
    """Stateless between calls except for what the caller passes: which request each row
    belongs to (`streams`), how many tokens it has drawn (`counters`) and, if the
    repetition penalty is on, its recent tokens."""

    def __init__(self, params: SamplerConfig, device):
        self.params = params
        self.device = torch.device(device)
        self._pinned = [None] * 4         # staging buffers for the per-row arrays, taken in turn
        self._events = [None] * 4
        self._turn = 0
        # the rows' arrays as they were last sent: rows that only advance together need no new copy
        self._rows_key = None
        self._rows_dev = None
        self._rows_counters = None
        self.h2d_bytes = 0                # bytes of per-row arrays copied to the device so far

    def _stage(self, meta: np.ndarray) -> torch.Tensor:
        """The per-row int32 arrays to the device, through pinned memory (no blocking copy)."""
        i = self._turn
        self._turn = (i + 1) % len(self._pinned)
        if self._events[i] is not None:
            self._events[i].synchronize()
        buf = self._pinned[i]
        if buf is None or buf.numel() < meta.size:
            buf = torch.empty(max(256, 2 * meta.size), dtype=torch.int32).pin_memory()
            self._pinned[i] = buf
        buf[:meta.size].copy_(torch.from_numpy(meta.reshape(-1)))
        self.h2d_bytes += meta.nbytes
        dev = buf[:meta.size].to(self.device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[i] = ev
        return dev

    def sample(self, logits: torch.Tensor, streams: list, counters: list, histories: list | None = None,
               out: torch.Tensor | None = None, mirror: torch.Tensor | None = None,
               newest: torch.Tensor | None = None) -> torch.Tensor:
        """logits: float32 [R, V] on the device (overwritten).  Returns int32 [R] on the device
        (`out` if given).  `mirror`: a pinned int32 host tensor that receives the tokens too,
        written by the kernel itself.  `newest`: int32 [R] on the device, each row's latest token
        when `histories` does not hold it yet (the host has not read it): it counts as the most
        recent id of the repetition window."""
        p = self.params
        rows = logits.shape[0]
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=self.device)
        recent = recent_count = None
        width = p.repetition_window if p.uses_history else 0
        keep = width - 1 if (width and newest is not None) else width       # ids of the window the host supplies
        if not width:
            # Without a history the rows' arrays are the streams and the counters.  The same rows one
            # draw further on keep the arrays they have on the device; the kernel adds the difference.
            key = tuple(streams)
            counters = list(counters)
            if key == self._rows_key and len(set(c - b for c, b in zip(counters, self._rows_counters))) <= 1:
                offset = counters[0] - self._rows_counters[0] if counters else 0
            else:
                meta = np.zeros(2 * rows, dtype=np.int32)
                meta[:rows] = streams
                meta[rows:] = counters
                self._rows_dev, self._rows_key, self._rows_counters, offset = self._stage(meta), key, counters, 0
            dev = self._rows_dev
            ops.sample(logits, out, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p, penalty=1.0, seed=p.seed,
                       row_stream=dev[:rows], row_counter=dev[rows:2 * rows], counter_offset=offset, mirror=mirror)
            return out
        # layout: streams [R], counters [R], history lengths [R], histories [R, width]: each contiguous
        meta = np.zeros(3 * rows + rows * width, dtype=np.int32)
        meta[:rows] = streams
        meta[rows:2 * rows] = counters
        if width:
            hist = meta[3 * rows:].reshape(rows, width)
            for r, h in enumerate(histories):
                tail = h[-keep:] if keep > 0 else []
                meta[2 * rows + r] = len(tail)
                hist[r, :len(tail)] = tail
        dev = self._stage(meta)
        row_stream, row_counter = dev[:rows], dev[rows:2 * rows]
        if width:
            recent_count = dev[2 * rows:3 * rows]
            recent = dev[3 * rows:].view(rows, width)
        ops.sample(logits, out, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p,
                   penalty=p.repetition_penalty, recent=recent, recent_count=recent_count, seed=p.seed,
                   row_stream=row_stream, row_counter=row_counter, mirror=mirror,
                   newest=newest if width else None)
        return out
