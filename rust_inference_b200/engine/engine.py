"""The engine: a model, its cache, and ONE step function.

`step` takes a batch of sequences with their next tokens (whole prompts of unequal
length, or one token each, or any continuation in between), runs exactly those tokens
as one packed batch against what earlier steps left in the cache, and returns float32
logits at the wanted places.  The reference's step is `Transformer::forward(token_id,
position, ...)` for one token of one sequence (transformer.rs:63-98), with the position
passed by the caller (model.rs:361-363); here the position comes from the slot's length.
"""
from __future__ import annotations

import dataclasses
from collections import OrderedDict

import numpy as np
import torch

from ..cache.sequence_cache import SequenceCache
from ..config.registry import get_architecture, load_spec
from ..weights.loader import random_tensors, read_model_tensors
from .context import StepContext, Workspace, pack_step
from .model import DecoderModel

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, found {dtype!r}") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"the engine runs on a CUDA device only; {device} was asked for")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; this library has no CPU path")
    return device


def resolve_max_seq_len(asked: int | None, limit: int) -> int:
    """The context length a run uses: the model's own (`max_position_embeddings`) unless a shorter
    one is asked for, as `--max-seq-len` overrides it in the reference (model.rs:142-144).  A
    longer one is an error: the model has no positions there."""
    if asked is None:
        return limit
    if asked <= 0:
        raise ValueError(f"max_seq_len must be positive, found {asked}")
    if asked > limit:
        raise ValueError(f"max_seq_len {asked} exceeds the model's max_position_embeddings {limit}")
    return int(asked)


class _PinnedRing:
    """Pinned host buffers for the per-step int32 arrays, reused round-robin; a buffer is
    rewritten only after the copy that read it has finished."""

    def __init__(self, n: int = 4):
        self.bufs = [None] * n
        self.events = [None] * n
        self.i = 0

    def stage(self, meta: np.ndarray, device) -> torch.Tensor:
        i = self.i
        self.i = (i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.bufs[i]
        if buf is None or buf.numel() < meta.size:
            buf = torch.empty(max(1024, 2 * meta.size), dtype=torch.int32).pin_memory()
            self.bufs[i] = buf
        buf[:meta.size].copy_(torch.from_numpy(meta))
        dev = buf[:meta.size].to(device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return dev


class Engine:
    def __init__(self, model: DecoderModel, *, max_tokens: int, max_seq_len: int | None = None,
                 n_slots: int | None = None, use_graphs: bool = True):
        self.model = model
        self.use_graphs = use_graphs and model.graph_safe()
        self._graphs: OrderedDict = OrderedDict()       # batch size -> DecodeGraph, least recently used first
        self._decode_logits = None                      # shared by batch sizes that have no graph yet
        self.device = require_cuda(model.device)
        self.dtype = model.dtype
        max_seq_len = resolve_max_seq_len(max_seq_len, model.spec.max_positions)
        self.cache = SequenceCache(model.cache_requests(), max_tokens=max_tokens, max_seq_len=max_seq_len,
                                   dtype=model.dtype, device=self.device, n_slots=n_slots)
        self.max_seq_len = self.cache.max_seq_len
        model.prepare(self.max_seq_len)
        self.workspace = Workspace(self.device)
        self._ring = _PinnedRing()
        self.h2d_bytes = 0          # bytes of step inputs copied to the device so far
        from ..kernels import ops
        if ops.checked_build():          # limits the kernels are not given as arguments (the last engine made sets them)
            ops.bounds_set_limits(model.spec.vocab_size, self.cache.n_slots, self.cache.n_pages)

    # ---- construction ----------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir: str, *, dtype="bfloat16", device="cuda", max_tokens: int = 8192,
                        max_seq_len: int | None = None, n_slots: int | None = None,
                        use_graphs: bool = True) -> "Engine":
        """Load a model folder (config.json + safetensors); the model class comes from
        config.json's architecture name."""
        device = require_cuda(device)
        config, spec = load_spec(model_dir)
        model = DecoderModel(spec, dtype=resolve_dtype(dtype), device=device)
        model.load(read_model_tensors(model_dir, model.declared_tensors(), spec.ignored_tensors))
        eng = cls(model, max_tokens=max_tokens, max_seq_len=max_seq_len, n_slots=n_slots, use_graphs=use_graphs)
        eng.config = config
        return eng

    @classmethod
    def from_random(cls, config, *, seed: int = 0, std: float = 0.02, norm_std: float = 0.0, dtype="bfloat16",
                    device="cuda", max_tokens: int = 8192, max_seq_len: int | None = None,
                    n_slots: int | None = None, use_graphs: bool = True) -> "Engine":
        """Random weights made on the device, without a folder (benchmarks)."""
        device = require_cuda(device)
        dtype = resolve_dtype(dtype)
        spec = get_architecture(config.architecture).build_spec(config)
        model = DecoderModel(spec, dtype=dtype, device=device)
        model.load(random_tensors(model.declared_tensors(), seed, std=std, matrix_dtype=dtype, device=device,
                                  norm_std=norm_std))
        eng = cls(model, max_tokens=max_tokens, max_seq_len=max_seq_len, n_slots=n_slots, use_graphs=use_graphs)
        eng.config = config
        return eng

    # ---- slots -------------------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def check_device_status(self) -> None:
        """Raise if a kernel gave up on a bounded wait since the last check (meaningful after a
        synchronisation point: a device-to-host read of the step's result); in the checked build
        (RI_B200_CHECK_BOUNDS=1) also if a kernel met an index outside its table."""
        if self.dtype == torch.bfloat16:
            from ..kernels import tcgen05
            tcgen05.check_status()
        from ..kernels import ops
        if ops.checked_build():
            found = ops.bounds_report()
            if found:
                raise ops.KernelError("the checked build found indices outside their tables: " + "; ".join(
                    f"{lib}: {what} ({index}, limit {limit}; {count} in all)" for lib, what, index, limit, count in found))

    # ---- the step ------------------------------------------------------------------
    def _check_batch(self, slots, tokens, wants):
        if len(slots) != len(tokens) or len(wants) != len(tokens):
            raise ValueError("step: slots, tokens and wants must have one entry per sequence")
        if not tokens:
            raise ValueError("step: an empty batch")
        if len(set(slots)) != len(slots):
            raise ValueError("step: a slot appears twice in one batch")
        vocab = self.model.spec.vocab_size
        for b, toks in enumerate(tokens):
            if len(toks) == 0:
                raise ValueError(f"step: sequence {b} brings no tokens")
            lo, hi = min(toks), max(toks)
            if lo < 0 or hi >= vocab:
                raise ValueError(f"step: sequence {b} has a token id outside [0, {vocab}): {lo if lo < 0 else hi}")

    def _stage(self, slots, tokens, wants):
        """Reserve cache room for the step and put its int32 arrays on the device."""
        self._check_batch(slots, tokens, wants)
        starts = self.cache.lengths(slots)
        self.cache.reserve([(s, st + len(t)) for s, st, t in zip(slots, starts, tokens)])
        meta, layout, sc = pack_step(starts, tokens, wants)
        o, c = layout["seq_slot"]
        meta[o:o + c] = slots
        dev = self._ring.stage(meta, self.device)
        self.h2d_bytes += meta.nbytes
        sc["host"] = (list(slots), starts, [len(t) for t in tokens])
        return dev, layout, sc

    def make_context(self, slots, tokens, wants) -> StepContext:
        dev, layout, sc = self._stage(slots, tokens, wants)

        def view(name):
            o, c = layout[name]
            return dev[o:o + c]

        return StepContext(
            n_tokens=sc["n_tokens"], n_seqs=sc["n_seqs"], token_ids=view("token_ids"),
            token_pos=view("token_pos"), token_seq=view("token_seq"), seq_slot=view("seq_slot"),
            seq_start=view("seq_start"), seq_len=view("seq_len"), cu_seqlens=view("cu_seqlens"),
            logit_rows=view("logit_rows"), n_logit_rows=sc["n_logit_rows"], max_new=sc["max_new"],
            max_len=sc["max_len"], all_single=sc["all_single"], page_table=self.cache.page_table,
            page_size=self.cache.page_size, dtype=self.dtype, device=self.device, workspace=self.workspace,
            host_slots=sc["host"][0], host_starts=sc["host"][1], host_counts=sc["host"][2])

    def step(self, slots: list, tokens: list, wants="last", borrow: bool = False, probe=None):
        """Run one step.

        slots[b]   cache slot of sequence b (from `alloc_slot`)
        tokens[b]  its next tokens (the whole prompt, or one token, or any run of tokens)
        wants      "last", "all", "none", or per sequence a list of places among its tokens
        Returns float32 logits [wanted places, vocab] on the device, in the order of the
        sequences and of their places; None if nothing is wanted.  With borrow=True the result
        may be a buffer that the next step overwrites (the generation loop consumes it at once).
        `probe`: an `engine.model.LayerProbe` that records the hidden state's statistics after every
        layer for chosen rows of the packed tokens (a debugging aid; the step then runs kernel by
        kernel, never as a captured graph)."""
        if wants == "last":
            wants = [[len(t) - 1] for t in tokens]
        elif wants == "all":
            wants = [list(range(len(t))) for t in tokens]
        elif wants == "none" or wants is None:
            wants = [[] for _ in tokens]
        decode = all(len(t) == 1 for t in tokens) and all(w == [0] for w in wants)
        with torch.cuda.device(self.device):
            if decode and self.use_graphs and probe is None:
                # one token per sequence, logits for each: the captured step of this batch size
                dev, _, _ = self._stage(slots, tokens, wants)
                logits = self._graph_for(len(slots)).run(dev)      # cleans up after itself if it raises
                if not borrow:
                    logits = logits.clone()
            else:
                ctx = self.make_context(slots, tokens, wants)
                try:
                    logits = self.model.forward(ctx, self.cache, probe=probe)
                except Exception:
                    self.workspace.rezero()          # accumulators a failed step may have left dirty
                    raise
        self.cache.advance(slots, [len(t) for t in tokens])
        return logits

    @staticmethod
    def _graph_key(n: int, sampler):
        # the seed lives on the device beside the draw counters: steps that differ in it share a capture
        return (n, None if sampler is None else dataclasses.replace(sampler, seed=0))

    def _graph_for(self, n: int, sampler=None):
        """The captured decode step of n sequences, with the sampler inside it if one is given (made
        on first use; call with the device current).  Only the most recently used ones are kept."""
        key = self._graph_key(n, sampler)
        graph = self._graphs.get(key)
        if graph is None:
            from .graphs import MAX_SIZES, DecodeGraph
            while len(self._graphs) >= MAX_SIZES:
                self._graphs.popitem(last=False)
            graph = self._graphs[key] = DecodeGraph(self, n, key[1])
        else:
            self._graphs.move_to_end(key)
        return graph

    def decode_graph(self, n: int, sampler=None):
        """The decode step of n sequences as the engine holds it (None if it has not been used yet)."""
        return self._graphs.get(self._graph_key(n, sampler))

    def shared_decode_logits(self, n: int) -> torch.Tensor:
        """float32 [n, vocab] for decode steps of batch sizes that have no buffer of their own yet; the
        next step overwrites it."""
        vocab = self.model.spec.vocab_size
        if self._decode_logits is None or self._decode_logits.numel() < n * vocab:
            self._decode_logits = torch.empty(n * vocab, dtype=torch.float32, device=self.device)
        return self._decode_logits[:n * vocab].view(n, vocab)

    def can_feed_from_device(self) -> bool:
        """True if decode steps replay a captured graph, so a step can take its tokens from a
        device tensor (`step_from_device`)."""
        return self.use_graphs

    def decode_token_buffer(self, n: int, sampler=None) -> torch.Tensor:
        """The int32 [n] device buffer from which the captured decode step of n sequences reads its
        tokens: a sampler that writes there feeds `step_from_device` without a copy."""
        with torch.cuda.device(self.device):
            return self._graph_for(n, sampler).ctx.token_ids

    def _enter_decode(self, graph, slots: list, streams=None, counters=None, seed=None) -> None:
        """Reserve a position for every sequence and make the graph's static arrays describe this step.
        When the step before was of the same sequences the arrays are already there (that step moved
        them on), and nothing is copied; otherwise they come from the host, together with the
        sampler's streams and draw counters if the step samples.  The token ids are left as they are."""
        n = len(slots)
        if len(set(slots)) != n:
            raise ValueError("step: a slot appears twice in one batch")
        starts = self.cache.lengths(slots)
        self.cache.reserve([(s, st + 1) for s, st in zip(slots, starts)])
        if graph.rows is not None:
            streams, counters = list(streams), list(counters)
        if graph.holds(slots, starts, streams, counters, seed):
            return
        meta, layout, _ = pack_step(starts, [[0]] * n, [[0]] * n)
        o, c = layout["seq_slot"]
        meta[o:o + c] = slots
        if graph.rows is not None:
            if len(streams) != n or len(counters) != n:
                raise ValueError("a step that samples needs a stream and a draw counter per sequence")
            seed_words = np.asarray([int(seed) & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64).view(np.int32)
            meta = np.concatenate([meta, np.asarray(streams, dtype=np.int32), np.asarray(counters, dtype=np.int32),
                                   seed_words])
        dev = self._ring.stage(meta, self.device)
        self.h2d_bytes += meta.nbytes
        graph.load_meta(dev, keep_tokens=True, slots=slots, starts=starts, streams=streams, counters=counters,
                        seed=seed)

    def _feed(self, graph, tokens_dev: torch.Tensor) -> None:
        if tokens_dev.numel() != graph.n_seqs or tokens_dev.dtype != torch.int32:
            raise ValueError("a decode step takes one int32 token per sequence")
        if tokens_dev.data_ptr() != graph.ctx.token_ids.data_ptr():       # else they are in place already
            graph.ctx.token_ids.copy_(tokens_dev, non_blocking=True)

    def step_from_device(self, slots: list, tokens_dev: torch.Tensor):
        """One decode step whose tokens (one per sequence, int32 [B]) are already on the device,
        for instance straight from the sampler: no host round trip between sampling and the next
        step.  Returns the step's logits [B, vocab] in a buffer the next step overwrites."""
        with torch.cuda.device(self.device):
            graph = self._graph_for(len(slots))
            self._enter_decode(graph, slots)
            self._feed(graph, tokens_dev)
            logits = graph.launch()
        self.cache.advance(slots, [1] * len(slots))
        return logits

    def can_sample_in_step(self, sampler_config) -> bool:
        """True if decode steps can hold this sampler (`step_and_sample_from_device`): captured steps,
        and options that need no token history."""
        return self.use_graphs and not sampler_config.uses_history

    def step_and_sample_from_device(self, slots: list, tokens_dev: torch.Tensor, sampler_config, streams: list,
                                    counters: list):
        """One decode step AND the sampling of its logits as one captured graph: feeds tokens_dev (int32
        [B] on the device), samples one token per sequence with `sampler_config` (row b draws its
        counters[b]-th number of stream streams[b]).  Returns (tokens on the device, the same in pinned
        host memory): the device buffer is the one the next step of these sequences reads, so passing it
        back costs nothing; the host buffer is valid once the step has finished (record an event behind
        this call and wait for it) and is reused four steps later.  While the same sequences go on, a
        step costs the host one graph launch: positions and draw counters move on on the device."""
        with torch.cuda.device(self.device):
            graph = self._graph_for(len(slots), sampler_config)
            self._enter_decode(graph, slots, streams, counters, sampler_config.seed)
            self._feed(graph, tokens_dev)
            graph.launch()
        self.cache.advance(slots, [1] * len(slots))
        return graph.ctx.token_ids, graph.last_tokens_host()

    def decode_steps(self, slots: list, first_tokens: list, n_steps: int, sampler_config=None,
                     on_step=None) -> torch.Tensor:
        """Device-resident decoding: n_steps steps of one token per sequence in which each
        sampled token is fed to the next step on the device, with no host round trip and no
        stop check in between.  Returns the sampled tokens, int32 [n_steps, B], on the device.
        The first step is fed `first_tokens`.  `on_step(i)` is called on the host just before step i
        is launched, everything it needs being in place (a benchmark records its event there)."""
        from ..sampling.params import SamplerConfig
        from .graphs import LOG_RING
        cfg = sampler_config or SamplerConfig.plain(temperature=0.0)
        if cfg.uses_history:
            raise ValueError("decode_steps keeps no token history: use it without a repetition penalty")
        if not self.use_graphs:
            raise RuntimeError("decode_steps replays a captured step; this engine runs without graphs "
                               "(a part of the model is not graph_safe, or graphs were switched off)")
        n = len(slots)
        self._check_batch(slots, [[t] for t in first_tokens], [[0]] * n)
        starts = self.cache.lengths(slots)
        self.cache.reserve([(s, st + n_steps) for s, st in zip(slots, starts)])      # all or nothing, up front
        streams = list(range(n))
        pieces = []
        with torch.cuda.device(self.device):
            graph = self._graph_for(n, cfg)
            first = self._ring.stage(np.asarray(first_tokens, dtype=np.int32), self.device)    # through the pinned ring: no allocation
            self.h2d_bytes += 4 * n
            done = 0
            while done < n_steps:
                run = min(LOG_RING, n_steps - done)
                for i in range(run):
                    self._enter_decode(graph, slots, streams, [done + i] * n, cfg.seed)
                    if done + i == 0:
                        self._feed(graph, first)
                    if on_step is not None:
                        on_step(done + i)
                    graph.launch()
                    self.cache.advance(slots, [1] * n)
                pieces.append(graph.logged_tokens(run))
                done += run
        return pieces[0] if len(pieces) == 1 else torch.cat(pieces)
