#!/usr/bin/env python3
"""Decode and prefill throughput of the library on one B200, with rooflines.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: a Qwen2.5-7B-sized dense decoder (28 layers, hidden 3584, 28 heads, 4 kv
heads, head_dim 128, intermediate 18944, vocabulary 152064, q/k/v biases, untied head)
with random bf16 weights, a batch of 8 sequences whose prompts have seeded random lengths
in 128..2048, in a cache of 8,192 positions per sequence.  A step is one decode step.

  value     decoded tokens per second over K timed decode steps, timed on the device
            (sampling on the device, each token fed to the next step without a host trip)
  e2e       the same through the Python entry point (`Model.generate`): host token ids in,
            host token ids out.  Every step's sampled tokens are read by the host (written to
            pinned memory by the step itself); what a step needs from the host goes up from
            pinned memory: the prompts, the arrays of a batch whenever its composition changes,
            new page-table entries.  While the same sequences go on a step's input token and
            positions are produced on the device, so the measured host-to-device bytes per step
            are few.  `ms_per_step_median` / `_worst` are taken from the host's clock, token to token.
  prefill   one 2,048-token prompt in one step
  roofline  bytes the decode step must read (every weight once, the cache of the live
            sequences) / step time, against the measured copy bandwidth
  points    decode tokens per second at batch 1 and batch 64 (their contexts and fractions of
            the copy bandwidth under `points_detail`)

The prompts' prefill runs the GPU into its power cap, and for some tens of milliseconds afterwards
decode steps take up to a tenth longer.  Every decode measurement therefore runs SETTLE_STEPS untimed
decode steps after its prefill, then the W warm-up steps, then the K timed ones.

Prints ONE JSON line.  Only one GPU is used: for --gpus > 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE configs[2]: the benchmark model (sizes of the model under test, not library constants)
MODEL = {
    "architectures": ["Qwen2ForCausalLM"], "hidden_size": 3584, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944,
    "vocab_size": 152064, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True,
    "tie_word_embeddings": False, "max_position_embeddings": 32768,
}
# further sizes of the same architecture, for --sizes (the default stays the benchmark model)
OTHER_SIZES = {
    "qwen2.5-7b": MODEL,
    "llama3-8b": {
        "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
        "vocab_size": 128256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "attention_bias": False,
        "tie_word_embeddings": False, "max_position_embeddings": 32768,
    },
    "qwen2.5-32b": {
        "architectures": ["Qwen2ForCausalLM"], "hidden_size": 5120, "num_hidden_layers": 64,
        "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 27648,
        "vocab_size": 152064, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True,
        "tie_word_embeddings": False, "max_position_embeddings": 32768,
    },
}
# the sizes the reference's README quotes its own (4-bit, CPU, batch 1) decode latencies for
OTHER_SIZES.update({
    "qwen2-0.5b": {
        "architectures": ["Qwen2ForCausalLM"], "hidden_size": 896, "num_hidden_layers": 24,
        "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 4864,
        "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True,
        "tie_word_embeddings": True, "max_position_embeddings": 32768,
    },
    "qwen2-1.5b": {
        "architectures": ["Qwen2ForCausalLM"], "hidden_size": 1536, "num_hidden_layers": 28,
        "num_attention_heads": 12, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 8960,
        "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True,
        "tie_word_embeddings": True, "max_position_embeddings": 32768,
    },
    "qwen2.5-3b": {
        "architectures": ["Qwen2ForCausalLM"], "hidden_size": 2048, "num_hidden_layers": 36,
        "num_attention_heads": 16, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 11008,
        "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True,
        "tie_word_embeddings": True, "max_position_embeddings": 32768,
    },
})
SIZE_NAMES = {"qwen2.5-7b": "Qwen2.5-7B-sized", "llama3-8b": "Llama-3-8B-sized", "qwen2.5-32b": "Qwen2.5-32B-sized",
              "qwen2-0.5b": "Qwen2-0.5B-sized", "qwen2-1.5b": "Qwen2-1.5B-sized", "qwen2.5-3b": "Qwen2.5-3B-sized"}
CONTEXT = 8192
PROMPT_MIN, PROMPT_MAX = 128, 2048
PREFILL_TOKENS = 2048
SETTLE_STEPS = 32
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
        except (KeyError, ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        fd, self.path = tempfile.mkstemp(prefix="bench_clocks_", suffix=".csv")
        os.close(fd)

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    # The prompts' prefill just before the timed steps runs the GPU into its power cap, and for some
    # tens of milliseconds afterwards decode steps take about a tenth longer: the default warm-up is
    # long enough to leave that behind.
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=32)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the model has (recorded)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--sizes", default="qwen2.5-7b", choices=sorted(OTHER_SIZES),
                    help="layer sizes of the model (default: the benchmark model)")
    ap.add_argument("--prompt-min", type=int, default=PROMPT_MIN, help="shortest prompt of the decode runs")
    ap.add_argument("--prompt-max", type=int, default=PROMPT_MAX, help="longest prompt of the decode runs")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS)
    ap.add_argument("--seq-len", type=int, default=CONTEXT, help="positions a sequence may reach (cache and rotary table)")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--kernel", default=None, help="time ONE kernel at the benchmark model's sizes instead "
                    "(qkv, qkv_split, o_proj, gate_up, down, lm_head, sample, attn_decode, attn_prefill, attn_prefill_mma, rmsnorm, rope)")
    ap.add_argument("--tokens", type=int, default=8, help="with --kernel: tokens in the step")
    ap.add_argument("--context", type=int, default=1024, help="with --kernel: cached positions per sequence")
    ap.add_argument("--once", action="store_true", help="with --kernel: launch the workload once, untimed (for ncu)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "yudono/rust-inference is a Rust crate (Cargo.toml, no Python packaging): pip cannot "
                          "install it, no Rust toolchain exists here, and its only GPU path is wgpu/WGSL, "
                          "which needs a graphics stack: unavailable on this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.kernel:
        from rust_inference_b200.kernels import microbench
        return microbench.main(args.kernel, OTHER_SIZES[args.sizes], args.tokens, args.context, args.once)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    import torch
    from rust_inference_b200 import SamplerConfig, config_from_dict
    from rust_inference_b200.api import Model
    from rust_inference_b200.kernels import ops

    peaks, peak_source = load_peaks()
    model_cfg = dict(OTHER_SIZES[args.sizes])
    prompt_min, prompt_max = max(1, args.prompt_min), max(args.prompt_min, args.prompt_max)
    prefill_tokens = max(1, args.prefill_tokens)
    layers_full = model_cfg["num_hidden_layers"]
    if args.layers:
        model_cfg["num_hidden_layers"] = args.layers
    cfg = config_from_dict(model_cfg)
    n_layers = cfg.num_hidden_layers

    total_steps = SETTLE_STEPS + warmup + steps + 2
    biggest = 64 if not args.skip_points else args.batch
    cache_tokens = max(biggest * (-(-(prompt_max + total_steps) // 64) * 64), prefill_tokens + 64) + 4096
    torch.cuda.set_device(0)
    t0 = time.time()
    seq_len = max(args.seq_len, prompt_max + total_steps, prefill_tokens)
    model_cfg["max_position_embeddings"] = max(model_cfg.get("max_position_embeddings", seq_len), seq_len)
    cfg = config_from_dict(model_cfg)
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_seq_len=seq_len,
                         max_tokens_in_cache=cache_tokens)
    engine = model.engine
    print(f"[bench] model ready in {time.time() - t0:.1f} s; cache {engine.cache.bytes() / 1e9:.2f} GB",
          file=sys.stderr, flush=True)

    weight_bytes = engine.model.weight_bytes(include_embedding=False)
    kv_bytes_per_token = n_layers * 2 * cfg.kv_dim * 2
    greedy = SamplerConfig.plain(temperature=0.0)

    def make_prompts(batch, seed):
        rng = random.Random(seed)
        lens = [rng.randint(prompt_min, prompt_max) for _ in range(batch)]
        return [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lens]

    def device_decode(batch, seed):
        """Prefill `batch` prompts, then time `steps` decode steps on the device."""
        prompts = make_prompts(batch, seed)
        slots = [engine.alloc_slot() for _ in prompts]
        for i in range(0, batch, 8):                       # prompts in groups, to bound scratch memory
            engine.step(slots[i:i + 8], prompts[i:i + 8], "none")
        first = [p[-1] for p in prompts]
        toks = engine.decode_steps(slots, first, SETTLE_STEPS + warmup, greedy)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # the first event goes onto the stream when the first timed step is about to be launched: what the
        # host does before that (reserving pages for all the steps, staging the first tokens) is no step
        toks = engine.decode_steps(slots, toks[-1].tolist(), steps, greedy,
                                   on_step=lambda i: e0.record() if i == 0 else None)
        e1.record()
        torch.cuda.synchronize()
        engine.check_device_status()
        ms = e0.elapsed_time(e1)
        graph = engine.decode_graph(batch, greedy)
        launches = steps * graph.launches                  # the captured kernels: model, sampler, the move to the next position
        ctx_tokens = sum(engine.cache.length(s) for s in slots) - batch * steps / 2.0
        for s in slots:
            engine.free_slot(s)
        step_bytes = weight_bytes + ctx_tokens * kv_bytes_per_token
        return {"tok_s": batch * steps / (ms * 1e-3), "ms_per_step": ms / steps, "launches": launches,
                "mean_ctx_tokens": ctx_tokens, "gb_s": step_bytes / (ms / steps * 1e-3) / 1e9}

    clocks = ClockSampler()
    clocks.start()

    main_run = device_decode(args.batch, seed=1)
    achieved_gbs = main_run["gb_s"]

    # ---- end to end through the Python entry point ----
    prompts = make_prompts(args.batch, seed=1)
    lead = SETTLE_STEPS + warmup
    results = model.generate(prompts, max_tokens=lead + steps + 1, sampler_config=greedy, stop_ids=(),
                             record_step_times=True)
    times = model.last_stats["step_times"]
    # times[0] is the prefill step; times[i] the i-th decode step's tokens on the host
    e2e_s = times[lead + steps] - times[lead]
    e2e_tok_s = args.batch * steps / e2e_s
    gaps = sorted((times[i + 1] - times[i]) * 1e3 for i in range(lead, lead + steps))
    # what went up from pinned memory during the whole call (prompts, the batch's arrays, new page-table
    # entries), averaged over its steps; the sampled tokens come down every step, written to pinned host
    # memory by the step itself
    h2d_per_step = model.last_stats["h2d_bytes"] / max(1, model.last_stats["steps"])
    d2h_per_step = args.batch * 4
    assert all(len(r.tokens) == lead + steps + 1 for r in results)

    # ---- prefill of 2,048 tokens ----
    rng = random.Random(7)
    prompt = [rng.randrange(cfg.vocab_size) for _ in range(prefill_tokens)]
    pre_ms = []
    for i in range(3 + 5):
        slot = engine.alloc_slot()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step([slot], [prompt], "last")
        e1.record()
        torch.cuda.synchronize()
        engine.free_slot(slot)
        if i >= 3:
            pre_ms.append(e0.elapsed_time(e1))
    pre_ms.sort()
    pre = pre_ms[len(pre_ms) // 2]
    t = prefill_tokens
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * cfg.hidden_size + cfg.hidden_size * cfg.q_dim \
        + 3 * cfg.intermediate_size * cfg.hidden_size
    flops = 2.0 * t * per_layer * n_layers + n_layers * 4.0 * t * t * cfg.q_dim / 2.0 \
        + 2.0 * cfg.vocab_size * cfg.hidden_size
    # frac: of the burst figure (a product timed alone).  The step is timed after the decode runs and three
    # untimed prefills, at the power cap; frac_of_sustained divides by the library's throughput in that state.
    prefill = {"value": t / (pre * 1e-3), "tokens": t, "ms": pre,
               "frac": flops / (pre * 1e-3) / (peaks["bf16_tflops"] * 1e12),
               "frac_of_sustained": flops / (pre * 1e-3) / (peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * 1e12)}

    points, points_detail = {}, {}
    if not args.skip_points:
        for b in (1, 64):
            r = device_decode(b, seed=100 + b)
            points[f"decode_b{b}"] = r["tok_s"]
            points_detail[f"decode_b{b}"] = {"ms_per_step": r["ms_per_step"], "mean_context": round(r["mean_ctx_tokens"] / b, 1),
                                             "gb_s": r["gb_s"], "frac": r["gb_s"] / peaks["hbm_gbs"]}
    engine.check_device_status()
    clock_info = clocks.stop()

    line = {
        "metric": f"decode tok/s @ batch {args.batch} ({SIZE_NAMES[args.sizes]} dense decoder, random bf16 weights, "
                  f"{seq_len:,}-position cache)",
        "value": main_run["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), seeded random token ids)",
        "impl": "ours",
        "config": {
            "model": f"{SIZE_NAMES[args.sizes]} dense decoder", "layers": n_layers, "layers_of_model": layers_full,
            "hidden_size": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate_size": cfg.intermediate_size, "vocab_size": cfg.vocab_size,
            "qkv_bias": cfg.attention_bias, "tied_embeddings": cfg.tie_word_embeddings,
            "global_batch": args.batch, "seq_len": seq_len, "prompt_lengths": f"uniform {prompt_min}-{prompt_max}",
            "mean_context": round(main_run["mean_ctx_tokens"] / args.batch, 1), "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights read once per step)", "peaks": peak_source,
            "settle_steps": SETTLE_STEPS,
        },
        "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": round(h2d_per_step, 1),
                "d2h_bytes_per_step": d2h_per_step, "ms_per_step_median": gaps[len(gaps) // 2],
                "ms_per_step_worst": gaps[-1]},
        "gpu_launches": main_run["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved_gbs / peaks["hbm_gbs"]},
        "points": points,
        "points_detail": points_detail,
        "clocks": clock_info,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
