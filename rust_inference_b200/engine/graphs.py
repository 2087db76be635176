"""CUDA graphs for decode steps.

A decode step of B sequences launches a few hundred small kernels; captured once per B
in a CUDA graph, it replays with one launch.  The graph reads the step's int32 arrays
from a static device buffer that is refilled before each replay and writes logits into a
static buffer; its scratch buffers are private, so nothing it points to ever moves.
Kernels size their grids from B and the cache geometry only, never from the current
lengths, so one capture serves every step of that batch size.

A batch size is captured only once it has been stepped a few times: a batch that loses a
sequence at every step passes through many sizes once, and capturing each (a second pass over
the model and a device synchronisation) would cost more than the launches it saves.
"""
from __future__ import annotations

import gc
import weakref

import numpy as np
import torch

from ..kernels import ops
from .context import StepContext, Workspace, pack_step


EAGER_STEPS = 2          # steps of a batch size that launch their kernels one by one before it is captured


class DecodeGraph:
    def __init__(self, engine, n_seqs: int):
        # a weak reference: the engine owns its graphs, and a cycle would leave both to the cyclic
        # collector, which may run in the middle of some later capture and destroy a CUDA graph there
        # (not permitted while a stream is capturing)
        self.engine = weakref.proxy(engine)
        self.n_seqs = n_seqs
        dev = engine.device
        # the layout of a step with one token per sequence depends on B only
        meta, self.layout, sc = pack_step([0] * n_seqs, [[0]] * n_seqs, [[0]] * n_seqs)
        self.meta_size = meta.size
        self.static_meta = torch.zeros(meta.size, dtype=torch.int32, device=dev)
        self.logits = torch.empty((n_seqs, engine.model.spec.vocab_size), dtype=torch.float32, device=dev)
        self.workspace = Workspace(dev)
        self.graph = None
        self.launches = 0             # kernels one replay launches
        self.eager_steps = 0

        def view(name):
            o, c = self.layout[name]
            return self.static_meta[o:o + c]

        self.ctx = StepContext(
            n_tokens=n_seqs, n_seqs=n_seqs, token_ids=view("token_ids"), token_pos=view("token_pos"),
            token_seq=view("token_seq"), seq_slot=view("seq_slot"), seq_start=view("seq_start"),
            seq_len=view("seq_len"), cu_seqlens=view("cu_seqlens"), logit_rows=view("logit_rows"),
            n_logit_rows=n_seqs, max_new=1, max_len=engine.max_seq_len, all_single=True,
            page_table=engine.cache.page_table, page_size=engine.cache.page_size, dtype=engine.dtype,
            device=dev, workspace=self.workspace, extras={"graph": True})

    def load_meta(self, meta_dev: torch.Tensor, keep_tokens: bool = False) -> None:
        """Refill the static arrays from this step's arrays (device, `pack_step` layout).  With
        keep_tokens the token ids already in the static buffer stay (the sampler wrote them)."""
        if keep_tokens:
            n = self.n_seqs                               # token_ids come first in the layout
            self.static_meta[n:].copy_(meta_dev[n:], non_blocking=True)
        else:
            self.static_meta.copy_(meta_dev, non_blocking=True)

    def launch(self) -> torch.Tensor:
        """Run the step over whatever the static arrays hold; returns the static logits buffer."""
        if self.graph is None:
            if self.eager_steps < EAGER_STEPS:
                # eagerly (the first time this also compiles, sizes scratch and caches tensor maps)
                self.eager_steps += 1
                before = ops.launch_count()
                self.engine.model.forward(self.ctx, self.engine.cache, self.logits)
                self.launches = ops.launch_count() - before
                return self.logits
            torch.cuda.synchronize(self.engine.device)
            g = torch.cuda.CUDAGraph()
            collecting = gc.isenabled()
            gc.disable()                  # no finalizer may touch CUDA while the stream is capturing
            try:
                with torch.cuda.graph(g):
                    self.engine.model.forward(self.ctx, self.engine.cache, self.logits)
            finally:
                if collecting:
                    gc.enable()
            self.graph = g
        self.graph.replay()
        return self.logits

    def run(self, meta_dev: torch.Tensor) -> torch.Tensor:
        self.load_meta(meta_dev)
        return self.launch()
