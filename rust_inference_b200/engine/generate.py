"""The generation loop above the step function.

The reference's loop (model.rs:332-478) serves one prompt: prefill token by token, then
sample, stop check, emit, forward, up to max_tokens times.  This one serves a list of
prompts of unequal length: as many as fit the cache start together as one batch (their
prompts in one step), then each live sequence gets one token per step; a sequence that
ends gives its slot back at once and the batch shrinks; when a batch is done the next
requests start, until all are served.

When the engine can take a step's tokens from the device, the loop looks one step ahead: the
next step is launched with the sampled tokens fed on the device, and the host reads the
tokens of the step before while it runs.  Which sequences end by length is known in advance;
a sequence that turns out to have sampled a stop token has simply run one step for nothing.

The loop here launches steps and reads tokens; what every request has generated, whether it goes on
and which requests fit the cache together is kept and decided by the native host runtime
(`engine/books.py` over `csrc/host_runtime.cpp`).

Kept from the reference: a sampled stop token ends the sequence and is not emitted
(model.rs:383-387); at most max_tokens tokens are generated (model.rs:373).  Changed: a
sequence that reaches the cache's max_seq_len ends with reason "length" instead of the
reference's panic (kv_cache.rs:54-59), and no forward pass is run for a token that
nothing will follow (the reference runs one, model.rs:431-438).
"""
from __future__ import annotations

import time
from dataclasses import dataclass

from .books import LIVE, REASONS, GenerationBooks


@dataclass
class GenerationResult:
    tokens: list
    finish_reason: str            # "stop" (a stop token was sampled) or "length"
    prompt_length: int


@dataclass
class _Live:
    index: int                    # which request (its tokens and history are in the books)
    slot: int
    prompt_length: int
    drawn: int = 0                # tokens sampled for it so far, read or not


class CudaLoopDevice:
    """The three things the look-ahead loop needs besides the engine and the sampler: host memory the
    device can write into, a mark on the stream that the host can wait for, and picking rows out of a
    token array.  A scripted stand-in (numpy arrays, marks that do nothing) lets the loop's decisions
    be tested without a GPU."""

    def host_buffer(self, n: int):
        import torch
        return torch.empty(n, dtype=torch.int32).pin_memory()

    def mark(self):
        import torch
        ev = torch.cuda.Event()
        ev.record()
        return ev

    def rows(self, tokens, keep: list):
        """tokens[keep] as a new array on the same side (device or pinned host) as `tokens`."""
        import torch
        idx = torch.tensor(keep, dtype=torch.long, device=tokens.device)
        return tokens[idx].contiguous()


class Generator:
    """engine: alloc_slot(), free_slot(slot), step(slots, tokens, "last") -> logits,
               max_seq_len, cache.pager (for admission)
       sampler: sample(logits, streams, counters, histories) -> int tokens (device or host)"""

    def __init__(self, engine, sampler, *, stop_ids=(), max_batch: int | None = None, device=None):
        self.engine = engine
        self.sampler = sampler
        self.device = device or CudaLoopDevice()     # what the look-ahead loop needs of the device
        self.stop_ids = frozenset(int(s) for s in stop_ids)
        self.max_batch = max_batch
        self.step_times = None        # set to a list to record when each step's tokens reached the host
        self.steps = 0                # model steps run (prefill and decode)
        self.d2h_bytes = 0            # bytes of sampled tokens read back

    def _to_host(self, tokens) -> list:
        if hasattr(tokens, "cpu"):
            tokens = tokens.cpu()
            self.d2h_bytes += tokens.numel() * tokens.element_size()
        return [int(t) for t in (tokens.tolist() if hasattr(tokens, "tolist") else tokens)]

    def _histories(self, seqs, keep=None):
        """The sampler's view of each sequence's past: the last ids of prompt and generated tokens."""
        window = getattr(getattr(self.sampler, "params", None), "repetition_window", 64)
        return self.books.recent([s.index for s in seqs], window if keep is None else keep)

    def _book(self, seqs, tokens, results) -> list:
        """Book one sampled token per sequence; returns the sequences that go on.  One that ends gives
        its result and its slot back at once."""
        status = self.books.book([s.index for s in seqs], tokens)
        still = []
        for s, st in zip(seqs, status):
            if st == LIVE:
                still.append(s)
                continue
            results[s.index] = GenerationResult(self.books.tokens(s.index), REASONS[st], s.prompt_length)
            self.engine.free_slot(s.slot)                            # the slot is free for the next batch
            s.slot = -1
        return still

    def _run_batch(self, live, prompts, max_tokens, results, uses_history) -> None:
        """Step, sample, read the tokens, decide, step again."""
        feed = [list(prompts[s.index]) for s in live]                # first step: whole prompts
        while True:
            logits = self.engine.step([s.slot for s in live], feed, "last", borrow=True)
            self.steps += 1
            sampled = self._to_host(self.sampler.sample(
                logits, [s.index for s in live], [s.drawn for s in live],
                self._histories(live) if uses_history else None))
            if hasattr(self.engine, "check_device_status"):
                self.engine.check_device_status()
            if self.step_times is not None:
                self.step_times.append(time.perf_counter())
            for s in live:
                s.drawn += 1
            fed = dict(zip((id(s) for s in live), sampled))
            live[:] = self._book(live, sampled, results)
            feed = [[fed[id(s)]] for s in live]
            if not live:
                return

    def _run_batch_ahead(self, live, prompts, max_tokens, results, uses_history=False) -> None:
        """The same with one step of lookahead: while the host reads the tokens sampled by step i,
        step i+1 already runs on them."""
        eng, dev = self.engine, self.device

        # A few host buffers the device can write to, taken in turn (at most two are awaited at any
        # time).  The sampling kernel writes its tokens there as well as to the device, so the host
        # needs no copy: it waits for the mark set behind the kernel.
        ring = [dev.host_buffer(len(live)) for _ in range(4)]
        turn = [0]

        books = self.books

        # A sampler that needs no token history can live inside the captured decode step: one graph
        # launch then runs the model, samples, and moves the step's arrays on for the next launch.
        in_step = self.sampler.params if (hasattr(eng, "can_sample_in_step") and hasattr(self.sampler, "params")
                                          and eng.can_sample_in_step(self.sampler.params)) else None

        def sample(logits, seqs, drawn, newest=None):
            host = ring[turn[0] % len(ring)][:len(seqs)]
            turn[0] += 1
            # straight into the buffer the next step of this batch size reads its tokens from, if the
            # whole batch will be stepped again at this size
            out = None
            if hasattr(eng, "decode_token_buffer") and all(books.goes_on([s.index for s in seqs], [d + 1 for d in drawn])):
                out = eng.decode_token_buffer(len(seqs), in_step) if in_step is not None else eng.decode_token_buffer(len(seqs))
            # With a repetition penalty the host's histories lack the token that was just fed (it has not
            # been read yet): the kernel takes that one from the device.  It reads `newest` before it writes
            # `out`, so the two may be the same buffer.
            # (the host's histories then give one id fewer, so that the window holds the same ids)
            hist = None
            if uses_history:
                window = getattr(self.sampler.params, "repetition_window", 64)
                hist = self._histories(seqs, window - 1 if (newest is not None and window > 0) else window)
            tokens_dev = self.sampler.sample(logits, [s.index for s in seqs], drawn, hist,
                                             out=out, mirror=host, newest=newest if uses_history else None)
            for s in seqs:
                s.drawn += 1
            self.d2h_bytes += len(seqs) * 4
            return tokens_dev, (host, dev.mark())

        logits = eng.step([s.slot for s in live], [list(prompts[s.index]) for s in live], "last", borrow=True)
        self.steps += 1
        pending = (list(live),) + sample(logits, live, [s.drawn for s in live])    # sequences, tokens on the device, (host copy, mark)
        while pending is not None:
            seqs, tokens_dev, (host, mark) = pending
            # who certainly goes on after the token just sampled (its drawn-th)?
            flags = books.goes_on([s.index for s in seqs], [s.drawn for s in seqs])
            rows = [i for i, on in enumerate(flags) if on]
            nxt = None
            if rows:
                ahead = [seqs[i] for i in rows]
                feed_dev = tokens_dev if len(rows) == len(seqs) else dev.rows(tokens_dev, rows)
                drawn = [s.drawn for s in ahead]
                if in_step is not None:
                    sampled, host2 = eng.step_and_sample_from_device([s.slot for s in ahead], feed_dev, in_step,
                                                                     [s.index for s in ahead], drawn)
                    for s in ahead:
                        s.drawn += 1
                    self.d2h_bytes += len(ahead) * 4
                    nxt = (ahead, sampled, (host2, dev.mark()))
                else:
                    logits = eng.step_from_device([s.slot for s in ahead], feed_dev)
                    nxt = (ahead,) + sample(logits, ahead, drawn, newest=feed_dev)
                self.steps += 1
            mark.synchronize()                                       # the earlier tokens; the step just launched keeps running
            if hasattr(eng, "check_device_status"):
                eng.check_device_status()
            if self.step_times is not None:
                self.step_times.append(time.perf_counter())
            going = self._book(seqs, host.tolist(), results)
            stopped = {id(s) for s in seqs} - {id(s) for s in going}
            if nxt is not None and stopped:
                # a sequence that sampled a stop token ran the step ahead for nothing: drop its row
                ahead, sampled, (host2, mark2) = nxt
                keep = [i for i, s in enumerate(ahead) if id(s) not in stopped]
                if not keep:
                    nxt = None
                elif len(keep) < len(ahead):
                    mark2.synchronize()
                    nxt = ([ahead[i] for i in keep], dev.rows(sampled, keep), (dev.rows(host2, keep), mark2))
            pending = nxt
        live[:] = [s for s in live if s.slot >= 0]

    # ---- the loop ---------------------------------------------------------------------
    def generate(self, prompts: list, max_tokens: int) -> list:
        results: list = [None] * len(prompts)
        uses_history = getattr(getattr(self.sampler, "params", None), "uses_history", False)
        self.books = books = GenerationBooks(max_tokens, self.engine.max_seq_len, self.stop_ids, uses_history)
        for p in prompts:
            books.add(p)                                             # refuses an empty or over-long prompt
        if max_tokens <= 0:
            return [GenerationResult([], "length", len(p)) for p in prompts]
        nxt = 0
        while nxt < len(prompts):
            count = books.admit(self.engine.cache.pager, nxt, self.max_batch)
            live = []
            for i in range(nxt, nxt + count):
                live.append(_Live(index=i, slot=self.engine.alloc_slot(), prompt_length=len(prompts[i])))
            nxt += count
            lookahead = (hasattr(self.sampler, "sample")
                         and getattr(self.engine, "can_feed_from_device", lambda: False)())
            try:
                if lookahead:
                    self._run_batch_ahead(live, prompts, max_tokens, results, uses_history)
                else:
                    self._run_batch(live, prompts, max_tokens, results, uses_history)
            finally:
                for s in live:                                       # only on an exception
                    if s.slot >= 0:
                        self.engine.free_slot(s.slot)
        return results
