"""The timeline build of the kernels (RI_B200_TIMELINE=1): every launch records when it came onto an SM and
when its wait for the kernel before ended.  It computes what the ordinary build computes, and its records
are in launch order with every wait ending after the one before.  Run in a process of its own: the build is
chosen when the package is imported."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent("""
    import sys, torch
    sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
    from conftest import make_model, random_tokens, rel_err
    import pathlib, tempfile
    from rust_inference_b200.engine.engine import Engine
    from rust_inference_b200.kernels import build, microbench, ops
    assert build.TIMELINE and ops.timeline_build() and "timeline" in build.library_path("elementwise")
    model = make_model(pathlib.Path(tempfile.mkdtemp()), "A", std=0.08)
    toks = random_tokens(80, model.cfg["vocab_size"], seed=1)
    want = model.plain_logits(toks)
    eng = Engine.from_pretrained(model.folder, dtype="bfloat16", max_tokens=512)
    s = eng.alloc_slot()
    head = eng.step([s], [toks[:70]], "all").cpu()
    tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in toks[70:79]])
    assert rel_err(torch.cat([head, tail]), want[:79]) <= 4e-2
    ops.timeline_read(strict=False)                     # what ran so far is not looked at
    eng.step([s], [[toks[79]]], "last")
    recs = ops.timeline_read()
    assert ops.timeline_read() == []                    # read once, then cleared
    layers = model.cfg["num_hidden_layers"]
    assert len(recs) >= 3 * layers, len(recs)           # at least the norms and the rotation of every layer
    names = {{}}
    kernels = []
    for r in recs:
        names.setdefault(r["module"], microbench._kernel_of_line(r["module"]))
        kernels.append(names[r["module"]](r["entry_line"]))
        assert r["entry_ns"] > 0 and r["wait_ns"] >= r["entry_ns"], r
    assert kernels[0] == "embed_gather_kernel" and sum(k.startswith("rmsnorm") for k in kernels) == 2 * layers + 1, kernels
    assert sum(k.startswith("rope_cache_write") for k in kernels) == layers, kernels
    entries = [r["entry_ns"] for r in recs]
    waits = [r["wait_ns"] for r in recs]
    assert entries == sorted(entries)
    assert waits == sorted(waits), "a kernel's wait ended before the wait of the kernel before it"
    print("timeline build ok", len(recs))
""")


def test_the_timeline_build_computes_the_same_and_records_every_launch_in_order():
    env = dict(os.environ, RI_B200_TIMELINE="1")
    env.pop("RI_B200_CHECK_BOUNDS", None)
    proc = subprocess.run([sys.executable, "-c", SCRIPT.format(root=ROOT, tests=os.path.join(ROOT, "tests"))],
                          env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0 and "timeline build ok" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-3000:]


def test_the_ordinary_build_keeps_no_timeline():
    from rust_inference_b200.kernels import build, ops
    if build.TIMELINE:
        pytest.skip("this process runs the timeline build")
    ops.rmsnorm(torch_ones(4, 32), torch_ones(32), 1e-5, torch_ones(4, 32))
    with pytest.raises(ops.KernelError, match="not a timeline build"):
        ops.timeline_read()


def torch_ones(*shape):
    import torch
    return torch.ones(*shape, device="cuda")
