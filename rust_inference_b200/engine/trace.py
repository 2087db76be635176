"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and owns no model code: it drives the same `Engine.step`, cache and
kernels that generation uses.  Steps arrive on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, `<out>/<step>.f32` receives the logits at the
wanted places (order of entries, then of `want`) as little-endian float32 [wanted, vocab].
After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    args = ap.parse_args(argv)

    from .engine import Engine   # imports torch; compiles kernels at first use

    os.makedirs(args.out, exist_ok=True)
    print(f"[trace_run] loading {args.model} ({args.dtype})", file=sys.stderr, flush=True)
    engine = Engine.from_pretrained(args.model, dtype=args.dtype, device="cuda", max_tokens=args.max_tokens)
    slots: dict = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step_no = rec["step"]
        entries = rec.get("entries", [])
        if entries:
            batch_slots, tokens, wants = [], [], []
            for e in entries:
                rid = e["id"]
                if rid not in slots:
                    slots[rid] = engine.alloc_slot()
                batch_slots.append(slots[rid])
                tokens.append([int(t) for t in e["tokens"]])
                wants.append([int(w) for w in e.get("want", [])])
            logits = engine.step(batch_slots, tokens, wants)
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                engine.check_device_status()
                arr.tofile(os.path.join(args.out, f"{step_no}.f32"))
        for rid in rec.get("end", []):
            if rid in slots:
                engine.free_slot(slots.pop(rid))
        print(f"done {step_no}", flush=True)
    return 0
