"""CUDA graphs for decode steps.

A decode step of B sequences launches a few hundred small kernels; captured once per B
in a CUDA graph, it replays with one launch.  The graph reads the step's int32 arrays
from a static device buffer that is refilled before each replay and writes logits into a
static buffer; its scratch buffers are private, so nothing it points to ever moves.
Kernels size their grids from B and the cache geometry only, never from the current
lengths, so one capture serves every step of that batch size.

A batch size is captured only once it has been stepped a few times: a batch that loses a
sequence at every step passes through many sizes once, and capturing each (a second pass over
the model and a device synchronisation) would cost more than the launches it saves.  Until
then a size owns nothing large: its first steps run on the engine's shared scratch and write
into the engine's shared logits buffer; the private logits buffer and scratch are made when
the size is about to be captured.  The engine keeps a bounded number of sizes (the least
recently used one goes first), so a batch that shrinks one sequence at a time does not pin a
logits buffer per size for the life of the engine.
"""
from __future__ import annotations

import gc
import weakref

import numpy as np
import torch

from ..kernels import ops
from .context import StepContext, Workspace, pack_step


EAGER_STEPS = 2          # steps of a batch size that run on the engine's shared buffers before it gets its own
MAX_SIZES = 8            # batch sizes an engine keeps graphs (or their beginnings) for


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
        self.logits = None            # private [n_seqs, vocab] float32, made before the capture
        self.workspace = None         # private scratch, made before the capture
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
            device=dev, workspace=engine.workspace, extras={"graph": True})

    def load_meta(self, meta_dev: torch.Tensor, keep_tokens: bool = False) -> None:
        """Refill the static arrays from this step's arrays (device, `pack_step` layout).  With
        keep_tokens the token ids already in the static buffer stay (the sampler wrote them)."""
        if keep_tokens:
            n = self.n_seqs                               # token_ids come first in the layout
            self.static_meta[n:].copy_(meta_dev[n:], non_blocking=True)
        else:
            self.static_meta.copy_(meta_dev, non_blocking=True)

    def _eager(self, logits: torch.Tensor) -> torch.Tensor:
        before = ops.launch_count()
        self.engine.model.forward(self.ctx, self.engine.cache, logits)
        self.launches = ops.launch_count() - before
        return logits

    def launch(self) -> torch.Tensor:
        """Run the step over whatever the static arrays hold; returns the logits in a buffer that a
        later step overwrites."""
        try:
            if self.graph is None:
                self.eager_steps += 1
                if self.eager_steps <= EAGER_STEPS:
                    # kernel by kernel, on the engine's shared scratch (the first time this also compiles
                    # and caches tensor maps)
                    self.ctx.workspace = self.engine.workspace
                    return self._eager(self.engine.shared_decode_logits(self.n_seqs))
                if self.workspace is None:
                    # this size stays: give it buffers of its own and run once more kernel by kernel,
                    # which sizes the scratch the capture will point to
                    self.workspace = Workspace(self.engine.device)
                    self.logits = torch.empty((self.n_seqs, self.engine.model.spec.vocab_size),
                                              dtype=torch.float32, device=self.engine.device)
                    self.ctx.workspace = self.workspace
                    return self._eager(self.logits)
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
        except Exception:
            self.abandon()
            raise

    def abandon(self) -> None:
        """After a step that did not finish: accumulators it may have left dirty hold zeros again, and
        a half-made capture is dropped (the size starts over with its own buffers)."""
        self.graph = None
        self.engine.workspace.rezero()
        if self.workspace is not None:
            self.workspace.rezero()

    def run(self, meta_dev: torch.Tensor) -> torch.Tensor:
        self.load_meta(meta_dev)
        return self.launch()
