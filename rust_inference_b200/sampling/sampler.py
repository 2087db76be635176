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

    def sample(self, logits: torch.Tensor, streams: list, counters: list, histories: list | None = None) -> torch.Tensor:
        """logits: float32 [R, V] on the device (overwritten).  Returns int32 [R] on the device."""
        p = self.params
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        recent = recent_count = None
        width = p.repetition_window if p.uses_history else 0
        meta = np.zeros((rows, 2 + 1 + width), dtype=np.int32)
        meta[:, 0] = streams
        meta[:, 1] = counters
        if width:
            for r, h in enumerate(histories):
                tail = h[-width:]
                meta[r, 2] = len(tail)
                meta[r, 3:3 + len(tail)] = tail
        dev = torch.from_numpy(meta).to(self.device, non_blocking=True)
        row_stream = dev[:, 0].contiguous()
        row_counter = dev[:, 1].contiguous()
        if width:
            recent_count = dev[:, 2].contiguous()
            recent = dev[:, 3:].contiguous()
        ops.sample(logits, out, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p,
                   penalty=p.repetition_penalty, recent=recent, recent_count=recent_count, seed=p.seed,
                   row_stream=row_stream, row_counter=row_counter)
        return out
