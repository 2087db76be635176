"""CUDA graphs for decode steps.

A decode step of B sequences launches a few hundred small kernels; captured once per B
in a CUDA graph, it replays with one launch.  The graph reads the step's int32 arrays
from a static device buffer and writes logits into a static buffer; its scratch buffers
are private, so nothing it points to ever moves.  Kernels size their grids from B and
the cache geometry only, never from the current lengths, so one capture serves every
step of that batch size.

The step ends with a small kernel that moves its own arrays on by one position
(`ops.advance_decode`), so the next step of the same sequences needs nothing from the host:
the static arrays are refilled only when the batch changes.  A step may also hold the
sampler (every option that needs no token history: greedy, temperature, top-k, top-p):
then the sampled tokens land in the step's own token buffer, where the next replay's
embedding reads them, and in a ring of pinned host buffers the generation loop reads from;
a decode step then costs the host one graph launch.

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
MAX_SIZES = 8            # batch sizes (times sampler settings) an engine keeps graphs, or their beginnings, for
HOST_RING = 4            # pinned buffers the sampled tokens of consecutive steps go to, in turn
LOG_RING = 256           # steps whose tokens stay readable on the device (`DecodeGraph.log`)


class DecodeGraph:
    def __init__(self, engine, n_seqs: int, sampler=None):
        """sampler: a `SamplerConfig` without token history to sample inside the step, or None."""
        # a weak reference: the engine owns its graphs, and a cycle would leave both to the cyclic
        # collector, which may run in the middle of some later capture and destroy a CUDA graph there
        # (not permitted while a stream is capturing)
        self.engine = weakref.proxy(engine)
        self.n_seqs = n_seqs
        self.sampler = sampler
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
        self.held = None              # [slots, lengths before the step, streams, draw counters] the static arrays describe now
        self.turn = 0                 # steps run: the host's copy of the device counter that picks the ring slots
        self.rows = self.turn_dev = self.host_ring = self.log = self.seed_dev = None
        if sampler is not None:
            if sampler.uses_history:
                raise ValueError("a step can only hold a sampler that needs no token history")
            # streams, then draw counters, then the seed (64 bits): another seed needs no other capture
            self.rows = torch.zeros(2 * n_seqs + 2, dtype=torch.int32, device=dev)
            self.seed_dev = self.rows[2 * n_seqs:].view(torch.int64)
            self.turn_dev = torch.zeros(1, dtype=torch.int32, device=dev)
            self.host_ring = torch.zeros((HOST_RING, n_seqs), dtype=torch.int32).pin_memory()
            self.log = torch.zeros((LOG_RING, n_seqs), dtype=torch.int32, device=dev)

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

    # ---- what the static arrays hold ------------------------------------------------------
    def holds(self, slots: list, starts: list, streams=None, counters=None, seed=None) -> bool:
        """True if the static arrays already describe a step of these slots at these lengths, drawing
        these numbers (the step before moved them on), so nothing has to come from the host."""
        h = self.held
        if h is None or h[0] != slots or h[1] != starts:
            return False
        return self.rows is None or (h[2] == streams and h[3] == counters and h[4] == seed)

    def load_meta(self, meta_dev: torch.Tensor, keep_tokens: bool = False, slots=None, starts=None,
                  streams=None, counters=None, seed=None) -> None:
        """Refill the static arrays from this step's arrays (device, `pack_step` layout, followed by the
        sampler's streams and draw counters if the step samples).  With keep_tokens the token ids
        already in the static buffer stay (the sampler wrote them)."""
        n, m = self.n_seqs, self.meta_size
        if keep_tokens:                                   # token_ids come first in the layout
            self.static_meta[n:].copy_(meta_dev[n:m], non_blocking=True)
        else:
            self.static_meta.copy_(meta_dev[:m], non_blocking=True)
        if self.rows is not None:
            if meta_dev.numel() < m + 2 * n + 2:
                raise ValueError("a step that samples needs its streams, draw counters and seed after the step's arrays")
            self.rows.copy_(meta_dev[m:m + 2 * n + 2], non_blocking=True)
        self.held = None
        if slots is not None:
            self.held = [list(slots), list(starts), list(streams) if streams is not None else None,
                         list(counters) if counters is not None else None, seed]

    # ---- running ------------------------------------------------------------------------------
    def _step(self, logits: torch.Tensor) -> None:
        """The kernels of one step: the model, the sampler if the step holds one, the move to the next position."""
        n, ctx = self.n_seqs, self.ctx
        self.engine.model.forward(ctx, self.engine.cache, logits)
        if self.sampler is not None:
            p = self.sampler
            ops.sample(logits, ctx.token_ids, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p, penalty=1.0,
                       seed=0, seed_dev=self.seed_dev, row_stream=self.rows[:n], row_counter=self.rows[n:2 * n],
                       counter_offset=0)
        ops.advance_decode(ctx.token_pos, ctx.seq_start, ctx.seq_len, ctx.token_ids,
                           draw_counter=self.rows[n:2 * n] if self.rows is not None else None, turn=self.turn_dev,
                           host_ring=self.host_ring, log_ring=self.log)

    def _eager(self, logits: torch.Tensor) -> torch.Tensor:
        before = ops.launch_count()
        self._step(logits)
        self.launches = ops.launch_count() - before
        return logits

    def launch(self) -> torch.Tensor:
        """Run the step over whatever the static arrays hold; returns the logits in a buffer that a
        later step overwrites (after a step that samples they have been consumed)."""
        try:
            out = self._launch()
        except Exception:
            self.abandon()
            raise
        if self.held is not None:                         # the step moved its arrays on by one position
            self.held[1] = [s + 1 for s in self.held[1]]
            if self.held[3] is not None:
                self.held[3] = [c + 1 for c in self.held[3]]
        self.turn += 1
        return out

    def _launch(self) -> torch.Tensor:
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
                    self._step(self.logits)
            finally:
                if collecting:
                    gc.enable()
            self.graph = g
        self.graph.replay()
        return self.logits

    def abandon(self) -> None:
        """After a step that did not finish: accumulators it may have left dirty hold zeros again, a
        half-made capture is dropped (the size starts over with its own buffers), and the static arrays
        count as unknown."""
        self.graph = None
        self.held = None
        self.engine.workspace.rezero()
        if self.workspace is not None:
            self.workspace.rezero()
        if self.turn_dev is not None:                     # the failed step may or may not have counted
            self.turn_dev.zero_()
            self.turn = 0

    def run(self, meta_dev: torch.Tensor) -> torch.Tensor:
        self.load_meta(meta_dev)
        return self.launch()

    # ---- a step that samples: where its tokens are --------------------------------------------
    def last_tokens_host(self) -> torch.Tensor:
        """The pinned int32 [n] buffer the step launched last writes its sampled tokens to (readable
        once that step has finished; the step after the next three overwrites it)."""
        return self.host_ring[(self.turn - 1) % HOST_RING]

    def logged_tokens(self, n_steps: int) -> torch.Tensor:
        """int32 [n_steps, n] on the device: what the last n_steps (at most LOG_RING) steps sampled."""
        if not 0 < n_steps <= LOG_RING:
            raise ValueError(f"the device keeps the tokens of the last {LOG_RING} steps")
        idx = torch.arange(self.turn - n_steps, self.turn, device=self.log.device) % LOG_RING
        return self.log.index_select(0, idx)
