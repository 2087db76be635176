"""Driving bin/trace_run from tests: build traces, feed them step by step, read the logits back."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Trace:
    """A list of steps plus, for every wanted row, which (request, position) it is."""

    def __init__(self):
        self.steps = []
        self.expect = {}          # step number -> [(request id, position)]

    def add(self, entries, end=()):
        """entries: [(id, tokens, want places, position of tokens[0])]"""
        n = len(self.steps)
        rows = []
        for rid, toks, want, pos0 in entries:
            rows += [(rid, pos0 + w) for w in want]
        self.steps.append({"step": n, "entries": [{"id": rid, "tokens": list(t), "want": list(w)}
                                                  for rid, t, w, _ in entries], "end": list(end)})
        if rows:
            self.expect[n] = rows
        return n

    def max_live_tokens(self):
        live, worst = {}, 0
        for s in self.steps:
            for e in s["entries"]:
                live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
            worst = max(worst, sum(-(-n // 64) * 64 for n in live.values()))
            for rid in s["end"]:
                live.pop(rid, None)
        return worst


def whole(requests: dict) -> Trace:
    """Each request alone and whole, one after another."""
    t = Trace()
    for rid, toks in requests.items():
        t.add([(rid, toks, range(len(toks)), 0)], end=[rid])
    return t


def last_decoded(requests: dict, n_last: int = 32) -> Trace:
    """Each request: all but the last n_last tokens in one step, then the rest one by one."""
    t = Trace()
    for rid, toks in requests.items():
        cut = len(toks) - n_last
        assert cut >= 1
        t.add([(rid, toks[:cut], range(cut), 0)])
        for i in range(cut, len(toks)):
            t.add([(rid, [toks[i]], [0], i)], end=[rid] if i == len(toks) - 1 else [])
    return t


def batches(groups: list, prompt_frac: float = 0.5) -> Trace:
    """groups: a list of {id: tokens}.  Each group starts together (the first part of every
    request in one step), then goes on by one token per step; shorter requests end earlier.
    The groups run one after another, so the later ones reuse what the earlier ones gave back."""
    t = Trace()
    for reqs in groups:
        cuts = {rid: max(1, int(len(toks) * prompt_frac)) for rid, toks in reqs.items()}
        ends = [rid for rid, toks in reqs.items() if cuts[rid] == len(toks)]
        t.add([(rid, toks[:cuts[rid]], range(cuts[rid]), 0) for rid, toks in reqs.items()], end=ends)
        live = {rid: cuts[rid] for rid in reqs if rid not in ends}
        while live:
            entries, ends = [], []
            for rid, pos in live.items():
                entries.append((rid, [reqs[rid][pos]], [0], pos))
                if pos + 1 == len(reqs[rid]):
                    ends.append(rid)
            t.add(entries, end=ends)
            live = {rid: pos + 1 for rid, pos in live.items() if rid not in ends}
    return t


def run_trace(model_dir: str, dtype: str, trace: Trace, out_dir: str, max_tokens: int | None = None,
              timeout: float = 600.0) -> dict:
    """Feed the trace to bin/trace_run step by step (the next step only after `done`).  Returns
    {step: float32 array [wanted, vocab]}."""
    max_tokens = max_tokens or trace.max_live_tokens()
    proc = subprocess.Popen(
        [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
         "--max-tokens", str(max_tokens)],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, bufsize=1)
    try:
        for s in trace.steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            if line.strip() != f"done {s['step']}":
                proc.stdin.close()
                err = proc.stderr.read()
                raise AssertionError(f"trace_run answered {line!r} to step {s['step']}\n{err[-3000:]}")
        proc.stdin.close()
        rc = proc.wait(timeout=timeout)
        err = proc.stderr.read()
        assert rc == 0, f"trace_run exited with {rc}\n{err[-3000:]}"
    finally:
        if proc.poll() is None:
            proc.kill()
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    out = {}
    for step in trace.expect:
        arr = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
        out[step] = torch.from_numpy(arr.reshape(-1, vocab).copy())
        assert out[step].shape[0] == len(trace.expect[step]), f"step {step}: wrong number of rows"
    extra = [f for f in os.listdir(out_dir) if f.endswith(".f32") and int(f[:-4]) not in trace.expect]
    assert not extra, f"files for steps in which nothing was wanted: {extra}"
    return out


def worst_error(trace: Trace, outputs: dict, plain: dict) -> tuple:
    """Largest per-row relative error against the plain logits, and where it is:
    (error, step, request id, position)."""
    worst = (0.0, None, None, None)
    for step, rows in trace.expect.items():
        got = outputs[step]
        for i, (rid, pos) in enumerate(rows):
            want = plain[rid][pos]
            err = float((got[i] - want).abs().max() / want.abs().max())
            if not err <= worst[0]:
                worst = (err, step, rid, pos)
    from conftest import note_error
    note_error(worst[0])
    return worst


def top_k_disagreements(trace: Trace, outputs: dict, plain: dict, k: int, tol: float) -> list:
    """Rows whose k largest logits are not the plain implementation's, among the rows where the plain
    order is decided by more than the tolerance could move it: [(step, request id, position)]."""
    from conftest import top_k_agrees
    bad = []
    for step, rows in trace.expect.items():
        for i, (rid, pos) in enumerate(rows):
            if not top_k_agrees(outputs[step][i], plain[rid][pos], k, tol):
                bad.append((step, rid, pos))
    return bad
