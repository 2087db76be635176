"""One kernel of the decoder at given sizes, timed on the device.

    python bench.py --kernel gate_up --tokens 8
    python bench.py --kernel attn_decode --tokens 64 --context 1024
    python bench.py --kernel step_parts --tokens 8      # what each kind of kernel costs INSIDE a decode step
    RI_B200_TIMELINE=1 python bench.py --kernel step_timeline --tokens 8     # the step kernel by kernel, as it overlaps
    python bench.py --kernel prefill_step --tokens 2048   # a prompt's step of the whole model, twelve times in a row

The operand that a step streams (weights, or the cache) is rotated over enough copies to
exceed L2, and the launches are replayed from a CUDA graph so that host launch cost is
not in the number.  Sizes default to the benchmark model of bench.py.  Used for the
profiles under profiles/ and for tuning.
"""
from __future__ import annotations

import json
import math

import torch

KERNELS = ("qkv", "qkv_split", "o_proj", "gate_up", "down", "lm_head", "sample", "attn_decode", "attn_prefill",
           "attn_prefill_mma", "rmsnorm", "rope", "step_parts", "step_timeline", "prefill_step")


def _graph_time(fn, launches_per_replay: int, reps: int = 10) -> float:
    """Microseconds per launch: fn() enqueues `launches_per_replay` launches; replayed `reps` times."""
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * launches_per_replay)


def run(kernel: str, model: dict, tokens: int, context: int = 1024, eager_only: bool = False) -> dict:
    from . import linear, ops, tcgen05
    from . import attention as attn
    dev = "cuda"
    h, inter, vocab = model["hidden_size"], model["intermediate_size"], model["vocab_size"]
    nh, nkv, hd = model["num_attention_heads"], model["num_key_value_heads"], model["head_dim"]
    qd, kvd = nh * hd, nkv * hd
    bf = torch.bfloat16

    def weights(n, k, copies):
        return [linear.Weight((torch.randn(n, k, device=dev) * 0.02).to(bf)) for _ in range(copies)]

    def copies_for(nbytes):
        return max(2, int(400e6 // nbytes) + 1)

    out = {"kernel": kernel, "tokens": tokens}
    if kernel in ("qkv", "qkv_split", "o_proj", "gate_up", "down", "lm_head"):
        n, k, mode = {"qkv": (qd + 2 * kvd, h, ops.EPI_STORE), "qkv_split": (qd + 2 * kvd, h, ops.EPI_RESIDUAL),
                      "o_proj": (h, qd, ops.EPI_RESIDUAL), "gate_up": (inter, h, ops.EPI_SILU_MUL),
                      "down": (h, inter, ops.EPI_RESIDUAL), "lm_head": (vocab, h, ops.EPI_STORE_F32)}[kernel]
        dual = mode == ops.EPI_SILU_MUL
        nbytes = n * k * 2 * (2 if dual else 1)
        c = copies_for(nbytes)
        ws = weights(n, k, c)
        w2s = weights(n, k, c) if dual else [None] * c
        x = (torch.randn(tokens, k, device=dev) * 0.5).to(bf)
        bias = torch.randn(n, device=dev) if kernel == "qkv" else None
        res = torch.zeros(tokens, n, device=dev, dtype=torch.float32 if mode in (ops.EPI_STORE_F32, ops.EPI_RESIDUAL) else bf)

        def fn():
            for i in range(c):
                tcgen05.gemm(x, ws[i], res, mode, bias=bias, w2=w2s[i])
        launches = c
        flops = 2.0 * tokens * n * k * (2 if dual else 1)
        out.update(n=n, k=k, bytes=nbytes + tokens * k * 2, flops=flops)
    elif kernel == "sample":
        # the reference's default sampling (temperature 0.8, top-k 40, top-p 0.95, penalty 1.1 over 64 ids) on
        # `tokens` rows of logits; the logits are overwritten, so every launch gets rows of its own
        c = max(4, int(200e6 // (tokens * vocab * 4)) + 1)
        rows = [torch.randn(tokens, vocab, device=dev) * 3 for _ in range(c)]
        fresh = [r.clone() for r in rows]
        toks = torch.empty(tokens, dtype=torch.int32, device=dev)
        stream = torch.arange(tokens, dtype=torch.int32, device=dev)
        counter = torch.zeros(tokens, dtype=torch.int32, device=dev)
        recent = torch.randint(0, vocab, (tokens, 64), dtype=torch.int32, device=dev)
        count = torch.full((tokens,), 64, dtype=torch.int32, device=dev)

        def fn():
            for i in range(c):
                rows[i].copy_(fresh[i])
                ops.sample(rows[i], toks, temperature=0.8, top_k=40, top_p=0.95, penalty=1.1, recent=recent,
                           recent_count=count, seed=12345, row_stream=stream, row_counter=counter)
        launches = c
        out.update(bytes=tokens * vocab * 4, flops=0.0, note="each launch follows a copy that restores its logits")
    elif kernel == "rmsnorm":
        x = torch.randn(tokens, h, device=dev)
        w = torch.ones(h, device=dev)
        y = torch.empty(tokens, h, device=dev, dtype=bf)

        def fn():
            for _ in range(20):
                ops.rmsnorm(x, w, 1e-6, y)
        launches = 20
        out.update(bytes=tokens * h * 6, flops=0.0)
    else:
        # a paged cache holding `context` positions per sequence (attn_decode: one new token per
        # sequence; attn_prefill: `tokens` new tokens of one sequence after `context - tokens` cached)
        page = 64
        n_seqs = tokens if kernel in ("attn_decode", "rope") else 1
        context = max(context, 1 if n_seqs > 1 else tokens)
        total = context
        pages_per = -(-total // page)
        layer_bytes = n_seqs * pages_per * nkv * page * hd * 2 * 2
        c = copies_for(layer_bytes) if kernel == "attn_decode" else 1
        kc = [torch.randn(n_seqs * pages_per, nkv, page, hd, device=dev).to(bf) for _ in range(c)]
        vc = [torch.randn(n_seqs * pages_per, nkv, page, hd, device=dev).to(bf) for _ in range(c)]
        table = torch.arange(n_seqs * pages_per, dtype=torch.int32, device=dev).view(n_seqs, pages_per)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        n_new = 1 if kernel in ("attn_decode", "rope") else tokens
        t_total = n_seqs * n_new
        slot, start = i32(list(range(n_seqs))), i32([total - n_new] * n_seqs)
        length, cu = i32([total] * n_seqs), i32([b * n_new for b in range(n_seqs + 1)])
        q = torch.randn(t_total, qd + 2 * kvd, device=dev).to(bf)
        o = torch.empty(t_total, qd, device=dev, dtype=bf)
        scale = 1.0 / math.sqrt(hd)
        if kernel == "attn_decode":
            name, splits = attn.decode_plan(n_seqs, nkv, pages_per * page, page)
            po = torch.empty(n_seqs * nh * splits * hd, device=dev)
            pml = torch.empty(n_seqs * nh * splits * 2, device=dev)
            decode_fn = attn.decode_kernel(name)
            out["decode_kernel"] = name

            def fn():
                for i in range(c):
                    decode_fn(q, q.shape[1], kc[i], vc[i], table, slot, length, cu, o, n_seqs=n_seqs,
                                         n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=page, scale=scale,
                                         window=0, n_splits=splits, part_o=po, part_ml=pml)
            launches = c
            out.update(bytes=layer_bytes, flops=4.0 * n_seqs * total * qd, splits=splits)
        elif kernel in ("attn_prefill", "attn_prefill_mma"):
            from . import attention_tc

            def fn():
                for _ in range(4):
                    if kernel == "attn_prefill":
                        attention_tc.prefill(q, kc[0], vc[0], table, slot, start, cu, o, n_seqs=1, max_new=n_new,
                                             n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=page, scale=scale)
                    else:
                        ops.attention_prefill(q, q.shape[1], kc[0], vc[0], table, slot, start, cu, o, n_seqs=1,
                                              max_new=n_new, n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                                              page_size=page, scale=scale, window=0)
            launches = 4
            first = total - n_new
            keys = sum(first + i + 1 for i in range(n_new))
            out.update(bytes=layer_bytes, flops=4.0 * keys * qd)
        else:   # rope + cache write from float32 accumulators
            from ..parts.rope import rope_tables
            cos, sin = rope_tables(hd, 1e6, total)
            cos, sin = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
            acc = torch.zeros(t_total, qd + 2 * kvd, device=dev)
            bias = torch.randn(qd + 2 * kvd, device=dev)
            pos, seq = i32([total - 1] * n_seqs), i32(list(range(n_seqs)))

            def fn():
                for _ in range(20):
                    ops.rope_cache_write_acc(acc, bias, o, cos, sin, pos, seq, slot, table, kc[0], vc[0], n_heads=nh,
                                             n_kv_heads=nkv, head_dim=hd, page_size=page, style=0, write_kv=True)
            launches = 20
            out.update(bytes=t_total * (qd + 2 * kvd) * 6, flops=0.0)
    if eager_only:
        fn()
        torch.cuda.synchronize()
        out["us"] = None
    else:
        us = _graph_time(fn, launches)
        out["us"] = us
        out["gb_per_s"] = out["bytes"] / us / 1e3
        out["tflop_per_s"] = out["flops"] / us / 1e6
    tcgen05.check_status()
    return out


def _decode_step_setup(model: dict, batch: int, prompt_min: int, prompt_max: int, room: int = 64):
    """The whole model with random weights, `batch` prompts of random lengths in its cache, and the
    device arrays of the decode step that follows them (with room for `room` such steps)."""
    import random
    from ..api import Model
    from ..config.registry import config_from_dict
    from ..engine.context import pack_step

    cfg = config_from_dict(dict(model))
    m = Model.random(cfg, seed=0, dtype="bfloat16", max_seq_len=8192, max_tokens_in_cache=batch * 2304 + 4096)
    eng = m.engine
    rng = random.Random(1)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.randint(prompt_min, prompt_max))] for _ in range(batch)]
    slots = [eng.alloc_slot() for _ in prompts]
    for i in range(0, batch, 8):
        eng.step(slots[i:i + 8], prompts[i:i + 8], "none")
    starts = eng.cache.lengths(slots)
    # every replay moves the step's positions on by one: room for all of them
    eng.cache.reserve([(s, st + room) for s, st in zip(slots, starts)])
    meta, layout, _ = pack_step(starts, [[5]] * batch, [[0]] * batch)
    o, c = layout["seq_slot"]
    meta[o:o + c] = slots
    rows = torch.cat([torch.arange(batch, dtype=torch.int32), torch.zeros(batch + 2, dtype=torch.int32)])   # streams, draw counters, seed
    meta_dev = torch.cat([torch.from_numpy(meta), rows]).cuda()
    return cfg, m, meta_dev


def _kernel_of_line(module: str):
    """line -> name of the `__global__` function of that module's source the line lies in."""
    import bisect
    import os
    import re
    from . import build
    with open(os.path.join(build.CSRC, build.MODULES[module])) as f:
        text = f.read()
    starts, names = [], []
    for mt in re.finditer(r"__global__\s+void\s+(?:__launch_bounds__\([^)]*\)\s*)?(\w+)\s*\(", text):
        starts.append(text.count("\n", 0, mt.start()) + 1)
        names.append(mt.group(1))

    def name(line: int) -> str:
        i = bisect.bisect_right(starts, line) - 1
        return names[i] if i >= 0 else f"{module}:{line}"
    return name


def step_timeline(model: dict, batch: int, prompt_min: int = 128, prompt_max: int = 2048, reps: int = 20) -> dict:
    """The captured decode step of `batch` sequences kernel by kernel, from the records the timeline
    build keeps (RI_B200_TIMELINE=1): for every kernel of a layer, averaged over the layers and over
    `reps` replays, `exclusive_us` (from the end of its wait for the kernel before to the end of the next
    kernel's wait: what it adds to the step), `resident_before_us` (how long it sat on an SM before
    the kernel before it finished: the prologue that programmatic dependent launch hides) and the
    places it marked, in microseconds after its wait ended."""
    from ..engine.graphs import DecodeGraph
    from ..sampling.params import SamplerConfig
    from . import ops, tcgen05

    if not ops.timeline_build():
        raise SystemExit("step_timeline needs the timeline build: run with RI_B200_TIMELINE=1")
    cfg, m, meta_dev = _decode_step_setup(model, batch, prompt_min, prompt_max, room=reps + 16)
    g = DecodeGraph(m.engine, batch, SamplerConfig.plain(0.0))
    for _ in range(4):                                      # three steps kernel by kernel, then the capture
        g.load_meta(meta_dev)
        g.launch()
    torch.cuda.synchronize()
    g.load_meta(meta_dev)
    for _ in range(3):
        g.graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        g.graph.replay()
    e1.record()
    torch.cuda.synchronize()
    step_us = e0.elapsed_time(e1) * 1e3 / 5
    ops.timeline_read(strict=False)                         # what ran so far is not looked at

    names: dict = {}
    runs = []
    for _ in range(reps):
        g.graph.replay()
        recs = ops.timeline_read()
        for r in recs:
            if r["module"] not in names:
                names[r["module"]] = _kernel_of_line(r["module"])
            r["kernel"] = names[r["module"]](r["entry_line"])
            r["start_ns"] = r["wait_ns"] or r["entry_ns"]
        runs.append(recs)
    tcgen05.check_status()
    n = len(runs[0])
    if any(len(r) != n for r in runs):
        raise RuntimeError("the replays recorded different numbers of kernels")
    seq = [r["kernel"] for r in runs[0]]
    layers = cfg.num_hidden_layers
    pre = period = None
    for p0 in range(0, 8):
        for k in range(2, 64):
            if p0 + layers * k <= n and all(seq[p0 + j] == seq[p0 + j + k] for j in range((layers - 1) * k)):
                pre, period = p0, k
                break
        if period:
            break
    if not period:
        raise RuntimeError(f"no repeating run of {layers} layers among {n} kernels: {seq[:40]}")

    def stats(index_sets):
        """Averages over the given record indices of every replay."""
        ex = res = 0.0
        ph = [0.0] * ops.TIMELINE_PHASES
        ph_n = [0] * ops.TIMELINE_PHASES
        cnt = 0
        for recs in runs:
            for i in index_sets:
                r = recs[i]
                if i + 1 < n:
                    ex += (recs[i + 1]["start_ns"] - r["start_ns"]) * 1e-3
                res += (r["start_ns"] - r["entry_ns"]) * 1e-3
                for k, t in enumerate(r["phases_ns"]):
                    if t:
                        ph[k] += (t - r["start_ns"]) * 1e-3
                        ph_n[k] += 1
                cnt += 1
        return {"exclusive_us": round(ex / cnt, 3), "resident_before_us": round(res / cnt, 3),
                "phases_us": [round(ph[k] / ph_n[k], 3) if ph_n[k] else None for k in range(ops.TIMELINE_PHASES)]}

    out = {"kernel": "step_timeline", "tokens": batch, "layers": layers, "kernels_per_step": n,
           "kernels_per_layer": period, "step_us_in_this_build": step_us,
           "recorded_span_us": sum((r[-1]["start_ns"] - r[0]["start_ns"]) for r in runs) * 1e-3 / reps,
           "before_layers": [], "layer": [], "after_layers": []}
    for i in range(pre):
        out["before_layers"].append({"kernel": seq[i], **stats([i])})
    for j in range(period):
        # the first layer follows the embedding and the last precedes the head: left out of the average
        idx = [pre + l * period + j for l in range(1, layers - 1)] or [pre + j]
        out["layer"].append({"kernel": seq[pre + j], "wait_line": runs[0][pre + j]["wait_line"], **stats(idx)})
    for i in range(pre + layers * period, n):
        out["after_layers"].append({"kernel": seq[i], **stats([i])})
    out["layer_us"] = round(sum(k["exclusive_us"] for k in out["layer"]), 3)
    stamps = sorted({r["start_ns"] for recs in runs for r in recs})
    out["timer_step_ns"] = min((b - a for a, b in zip(stamps, stamps[1:])), default=0)
    return out


def prefill_step(model: dict, tokens: int, reps: int = 12) -> dict:
    """One prompt of `tokens` tokens through the whole model, `reps` times in a row in a process that has
    run nothing else: the first steps find the GPU idle and cool, the later ones run at its power cap."""
    import random
    from ..api import Model
    from ..config.registry import config_from_dict

    cfg = config_from_dict(dict(model))
    m = Model.random(cfg, seed=0, dtype="bfloat16", max_seq_len=max(8192, tokens), max_tokens_in_cache=tokens + 4096)
    eng = m.engine
    rng = random.Random(7)
    prompt = [rng.randrange(cfg.vocab_size) for _ in range(tokens)]
    times = []
    for _ in range(reps):
        slot = eng.alloc_slot()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([slot], [prompt], "last")
        e1.record()
        torch.cuda.synchronize()
        eng.free_slot(slot)
        times.append(round(e0.elapsed_time(e1), 3))
    eng.check_device_status()
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * cfg.hidden_size + cfg.hidden_size * cfg.q_dim \
        + 3 * cfg.intermediate_size * cfg.hidden_size
    flops = 2.0 * tokens * per_layer * cfg.num_hidden_layers + cfg.num_hidden_layers * 4.0 * tokens * tokens * cfg.q_dim / 2.0 \
        + 2.0 * cfg.vocab_size * cfg.hidden_size
    return {"kernel": "prefill_step", "tokens": tokens, "ms": times, "flops": flops,
            "tflop_per_s": [round(flops / (t * 1e-3) * 1e-12, 1) for t in times]}


def step_parts(model: dict, batch: int, prompt_min: int = 128, prompt_max: int = 2048) -> dict:
    """What each kind of kernel costs inside a decode step of `batch` sequences of the whole model: the
    captured step (model, greedy sampler, move to the next position) is timed as it is and again with
    one kind of kernel left out; the difference is that kind's share with everything that overlaps it
    (programmatic dependent launch, tails and ramps) counted as it falls.  Results are microseconds
    per step; the step without a kernel computes nothing meaningful and is only timed."""
    from ..engine.graphs import DecodeGraph
    from ..parts import attention as attention_part
    from ..sampling.params import SamplerConfig
    from . import ops, tcgen05

    cfg, m, meta_dev = _decode_step_setup(model, batch, prompt_min, prompt_max)
    eng = m.engine
    greedy = SamplerConfig.plain(0.0)

    def time_step(sampler=greedy, reps=30):
        g = DecodeGraph(eng, batch, sampler)
        for _ in range(4):                                  # three steps kernel by kernel, then the capture
            g.load_meta(meta_dev)
            g.launch()
        torch.cuda.synchronize()
        for _ in range(5):
            g.graph.replay()
        g.load_meta(meta_dev)                               # back to the first position
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    def without(patches):
        saved = [(obj, attr, getattr(obj, attr)) for obj, attr, _ in patches]
        for obj, attr, new in patches:
            setattr(obj, attr, new)
        try:
            return time_step()
        finally:
            for obj, attr, old in saved:
                setattr(obj, attr, old)

    real_gemm = tcgen05.gemm

    def gemm_except(skip):
        def gemm(x, w, out, mode, ctx=None, bias=None, w2=None, split_k=None):
            return out if skip(w, mode) else real_gemm(x, w, out, mode, ctx, bias=bias, w2=w2, split_k=split_k)
        return gemm

    noop = lambda *a, **k: None
    qd, kvd, h, inter = cfg.q_dim, cfg.kv_dim, cfg.hidden_size, cfg.intermediate_size
    full = time_step()
    out = {"kernel": "step_parts", "tokens": batch, "layers": cfg.num_hidden_layers, "step_us": full, "without_us": {}}
    cases = {
        "sampler": lambda: time_step(sampler=None),
        "attention": lambda: without([(attention_part.attn_kernels, "attention", noop)]),
        "rope_cache_write": lambda: without([(ops, "rope_cache_write_acc", noop), (ops, "rope_cache_write", noop)]),
        "rmsnorm": lambda: without([(ops, "rmsnorm", lambda x, w, eps, out, rows=None: out)]),
        "qkv_gemm": lambda: without([(tcgen05, "gemm", gemm_except(lambda w, mode: w.n == qd + 2 * kvd and w.k == h))]),
        "o_gemm": lambda: without([(tcgen05, "gemm", gemm_except(lambda w, mode: w.n == h and w.k == qd and mode == ops.EPI_RESIDUAL))]),
        "gate_up_gemm": lambda: without([(tcgen05, "gemm", gemm_except(lambda w, mode: mode == ops.EPI_SILU_MUL))]),
        "down_gemm": lambda: without([(tcgen05, "gemm", gemm_except(lambda w, mode: w.k == inter))]),
        "lm_head": lambda: without([(tcgen05, "gemm", gemm_except(lambda w, mode: mode == ops.EPI_STORE_F32))]),
        "mixer (norm, qkv, rope, attention, o)": lambda: without([(attention_part.GQAttention, "forward", noop)]),
    }
    for name, run in cases.items():
        out["without_us"][name] = run()
    out["share_us"] = {name: full - t for name, t in out["without_us"].items()}
    tcgen05.check_status()
    return out


def main(kernel: str, model: dict, tokens: int, context: int, eager_only: bool = False) -> int:
    if kernel not in KERNELS:
        print(f"unknown kernel {kernel!r}; choose from {', '.join(KERNELS)}")
        return 2
    if kernel == "step_parts":
        print(json.dumps(step_parts(model, tokens)))
        return 0
    if kernel == "step_timeline":
        print(json.dumps(step_timeline(model, tokens)))
        return 0
    if kernel == "prefill_step":
        print(json.dumps(prefill_step(model, tokens)))
        return 0
    print(json.dumps(run(kernel, model, tokens, context, eager_only)))
    return 0
