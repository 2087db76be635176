"""The command line as a user starts it: `bin/gguf-infer` as a process on a model folder and in the
random-weights mode; its standard output is the generated token ids, one line per prompt."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_impl
from conftest import TINY, random_tokens

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "bin", "gguf-infer")


def _run(*args, timeout=600):
    proc = subprocess.run([sys.executable, CLI, *[str(a) for a in args]], capture_output=True, text=True, timeout=timeout)
    return proc.returncode, proc.stdout, proc.stderr


def test_greedy_generation_from_a_model_folder(model_factory):
    model = model_factory("A", std=0.08)
    prompts = [random_tokens(n, model.cfg["vocab_size"], seed=60 + n) for n in (4, 13, 1)]
    args = ["--model", model.folder, "--temperature", "0", "--repetition-penalty", "1", "--max-tokens", "7",
            "--dtype", "float32"]
    for p in prompts:
        args += ["--prompt", ",".join(str(t) for t in p)]
    args += ["--stop-ids", ""]
    rc, out, err = _run(*args)
    assert rc == 0, err[-2000:]
    lines = [l for l in out.splitlines() if l.strip()]
    want = [plain_impl.greedy_generate(model.weights, model.cfg, p, 7) for p in prompts]
    assert [[int(t) for t in l.split()] for l in lines] == want
    assert "21 tokens in" in err and "finish: length, length, length" in err
    # a stop id given on the command line ends a sequence and is not printed (model.rs:383-387)
    stop = want[1][2]
    rc, out, err = _run(*args[:-2], "--stop-ids", str(stop))
    assert rc == 0, err[-2000:]
    got = [[int(t) for t in l.split()] for l in out.split("\n")[:3]]
    for g, w in zip(got, want):
        assert g == (w[:w.index(stop)] if stop in w else w)


def test_the_default_sampling_is_the_references(model_factory):
    """No sampling flags: temperature 0.8, top-k 40, top-p 0.95, penalty 1.1 over 64 ids, seed 12345
    (main.rs:65-69, :187-188): the same command twice prints the same ids; another seed prints others."""
    model = model_factory("B", std=0.08)
    base = ["--model", model.folder, "--prompt", "5 6 7 8", "-n", "12", "--stop-ids", ""]
    rc, a, err = _run(*base)
    assert rc == 0, err[-2000:]
    rc, b, _ = _run(*base)
    rc2, c, _ = _run(*base, "-s", "7")
    assert rc == 0 and rc2 == 0
    assert a == b and len(a.split()) == 12
    assert a != c


def test_random_weights_mode_with_statistics(tmp_path):
    cfg = dict(TINY["B"])
    path = tmp_path / "config.json"
    path.write_text(json.dumps(cfg))
    rc, out, err = _run("--random-config", path, "--weights-seed", 3, "--random-prompts", "3:2:9", "--slots", 2,
                        "-n", 4, "-t", 0, "--repetition-penalty", 1, "--print-logits-topk", 3, "--dump-layer-stats",
                        "--dtype", "float32", "--stop-ids", "", "--bench")
    assert rc == 0, err[-2000:]
    lines = [l.split() for l in out.splitlines() if l.strip()]
    assert len(lines) == 3 and all(len(l) == 4 for l in lines)
    stats = json.loads(err.strip().splitlines()[-1])
    assert stats["generated_tokens"] == 12 and stats["tokens_per_second"] > 0 and stats["weight_bytes"] > 0
    # three prompts: for each the statistics of every layer and of the final norm, then the top logits
    assert err.count("[L0] min=") == 3 and err.count("[L2] min=") == 3 and err.count("[FNL] min=") == 3
    assert err.count("top logits") == 3
    # the first generated token is the largest logit printed for its prompt
    tops = [l for l in err.splitlines() if "top logits" in l]
    for gen, top in zip(lines, tops):
        assert int(top.split("top logits")[1].split()[0].split(":")[0]) == int(gen[0])


def test_errors_exit_with_one(tmp_path):
    rc, _, err = _run("--model", tmp_path / "nothing", "--prompt", "1")
    assert rc == 1 and "not found" in err and "Usage: gguf-infer" in err      # main.rs:173-177
    (tmp_path / "m").mkdir()
    rc, _, err = _run("--model", tmp_path / "m", "--prompt", "1")
    assert rc == 1 and "Failed to load model" in err                           # main.rs:257-263


def test_layer_statistics_match_the_plain_implementation(model_factory):
    from rust_inference_b200 import Model
    model = model_factory("B", std=0.08)
    toks = random_tokens(9, model.cfg["vocab_size"], seed=2)
    want = []
    plain_impl.forward(model.weights, model.cfg, toks, stats=want)
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 4e-2)):
        got = []
        Model.load(model.folder, dtype=dtype, max_tokens_in_cache=256).logits(toks, "last", layer_stats=got)
        assert [g[0] for g in got] == [w[0] for w in want] == ["L0", "L1", "L2", "FNL"]
        for (_, g), (_, w) in zip(got, want):
            scale = max(abs(w["min"]), abs(w["max"]))
            for key in ("min", "max", "mean"):
                assert abs(g[key] - w[key]) <= tol * scale, (dtype, key)
            assert max(abs(a - b) for a, b in zip(g["first"], w["first"])) <= tol * scale
