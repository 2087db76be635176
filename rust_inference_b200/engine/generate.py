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

Kept from the reference: a sampled stop token ends the sequence and is not emitted
(model.rs:383-387); at most max_tokens tokens are generated (model.rs:373).  Changed: a
sequence that reaches the cache's max_seq_len ends with reason "length" instead of the
reference's panic (kv_cache.rs:54-59), and no forward pass is run for a token that
nothing will follow (the reference runs one, model.rs:431-438).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field


@dataclass
class GenerationResult:
    tokens: list
    finish_reason: str            # "stop" (a stop token was sampled) or "length"
    prompt_length: int


@dataclass
class _Live:
    index: int                    # which request
    slot: int
    prompt_length: int
    tokens: list = field(default_factory=list)
    history: list = field(default_factory=list)


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

    # ---- admission: which requests start together ---------------------------------
    def _admit(self, prompts, first: int, max_tokens: int) -> int:
        """How many requests, starting at `first`, fit the cache together.  Every admitted
        request has pages for its prompt plus all the tokens it may generate, so a batch
        never runs out of room half way."""
        pager = self.engine.cache.pager
        page = pager.page_size
        free_pages, free_slots = pager.free_page_count(), pager.free_slot_count()
        n = 0
        while first + n < len(prompts):
            if self.max_batch is not None and n >= self.max_batch:
                break
            length = min(len(prompts[first + n]) + max_tokens, self.engine.max_seq_len)
            need = -(-length // page)
            if need > free_pages or free_slots == 0:
                break
            free_pages -= need
            free_slots -= 1
            n += 1
        if n == 0:
            raise RuntimeError(
                f"request {first} (prompt of {len(prompts[first])} tokens, up to {max_tokens} more) "
                f"does not fit the cache even alone")
        return n

    def _to_host(self, tokens) -> list:
        if hasattr(tokens, "cpu"):
            tokens = tokens.cpu()
            self.d2h_bytes += tokens.numel() * tokens.element_size()
        return [int(t) for t in (tokens.tolist() if hasattr(tokens, "tolist") else tokens)]

    def _finish_or_keep(self, s, tok, max_tokens, results) -> bool:
        """Book one sampled token of sequence s; returns True if s goes on."""
        reason = None
        if tok in self.stop_ids:
            reason = "stop"                                          # not emitted, not fed back
        else:
            s.tokens.append(tok)
            if len(s.tokens) >= max_tokens:
                reason = "length"
            elif s.prompt_length + len(s.tokens) > self.engine.max_seq_len:
                reason = "length"                                    # no position left to feed it at
        if reason is None:
            return True
        results[s.index] = GenerationResult(s.tokens, reason, s.prompt_length)
        self.engine.free_slot(s.slot)                                # the slot is free for the next batch
        s.slot = -1
        return False

    def _run_batch(self, live, prompts, max_tokens, results, uses_history) -> None:
        """Step, sample, read the tokens, decide, step again."""
        feed = [list(prompts[s.index]) for s in live]                # first step: whole prompts
        while True:
            logits = self.engine.step([s.slot for s in live], feed, "last", borrow=True)
            self.steps += 1
            sampled = self._to_host(self.sampler.sample(
                logits, [s.index for s in live], [len(s.tokens) for s in live],
                [s.history for s in live] if uses_history else None))
            if hasattr(self.engine, "check_device_status"):
                self.engine.check_device_status()
            if self.step_times is not None:
                self.step_times.append(time.perf_counter())
            still, feed = [], []
            for s, tok in zip(list(live), sampled):
                if self._finish_or_keep(s, tok, max_tokens, results):
                    if uses_history:
                        s.history.append(tok)
                    still.append(s)
                    feed.append([tok])
            live[:] = still
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

        def goes_on(s, drawn) -> bool:
            """Will s certainly be stepped again after its next token (its drawn-th)?  Length limits are
            known in advance; stop tokens are not."""
            return drawn < max_tokens and s.prompt_length + drawn <= eng.max_seq_len

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
            if hasattr(eng, "decode_token_buffer") and all(goes_on(s, d + 1) for s, d in zip(seqs, drawn)):
                out = eng.decode_token_buffer(len(seqs), in_step) if in_step is not None else eng.decode_token_buffer(len(seqs))
            # With a repetition penalty the host's histories lack the token that was just fed (it has not
            # been read yet): the kernel takes that one from the device.  It reads `newest` before it writes
            # `out`, so the two may be the same buffer.
            tokens_dev = self.sampler.sample(logits, [s.index for s in seqs], drawn,
                                             [s.history for s in seqs] if uses_history else None,
                                             out=out, mirror=host, newest=newest if uses_history else None)
            self.d2h_bytes += len(seqs) * 4
            return tokens_dev, (host, dev.mark())

        logits = eng.step([s.slot for s in live], [list(prompts[s.index]) for s in live], "last", borrow=True)
        self.steps += 1
        pending = (list(live),) + sample(logits, live, [len(s.tokens) for s in live])    # sequences, tokens on the device, (host copy, mark)
        while pending is not None:
            seqs, tokens_dev, (host, mark) = pending
            rows = [i for i, s in enumerate(seqs) if goes_on(s, len(s.tokens) + 1)]
            nxt = None
            if rows:
                ahead = [seqs[i] for i in rows]
                feed_dev = tokens_dev if len(rows) == len(seqs) else dev.rows(tokens_dev, rows)
                drawn = [len(s.tokens) + 1 for s in ahead]
                if in_step is not None:
                    sampled, host2 = eng.step_and_sample_from_device([s.slot for s in ahead], feed_dev, in_step,
                                                                     [s.index for s in ahead], drawn)
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
            stopped = set()
            for s, tok in zip(seqs, host.tolist()):
                if not self._finish_or_keep(s, int(tok), max_tokens, results):
                    stopped.add(id(s))
                elif uses_history:
                    s.history.append(int(tok))
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
        for i, p in enumerate(prompts):
            if len(p) == 0:
                raise ValueError(f"request {i}: empty prompt")
            if len(p) > self.engine.max_seq_len:
                raise ValueError(f"request {i}: prompt of {len(p)} tokens exceeds max_seq_len "
                                 f"{self.engine.max_seq_len}")
        results: list = [None] * len(prompts)
        if max_tokens <= 0:
            return [GenerationResult([], "length", len(p)) for p in prompts]
        uses_history = getattr(getattr(self.sampler, "params", None), "uses_history", False)
        nxt = 0
        while nxt < len(prompts):
            count = self._admit(prompts, nxt, max_tokens)
            live = []
            for i in range(nxt, nxt + count):
                live.append(_Live(index=i, slot=self.engine.alloc_slot(), prompt_length=len(prompts[i]),
                                  history=list(prompts[i]) if uses_history else []))
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
