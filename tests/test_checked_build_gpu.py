"""The checked build of the kernels (RI_B200_CHECK_BOUNDS=1): indices that reach memory through a table
are compared with their limits, recorded and skipped when outside.  It stands where a memory checker
would: it runs the ordinary tests' kind of work and must stay silent, and it must speak when it is fed a
bad index.  The bad indices below are only ever given to the checked build, which does not follow them.
Run in a process of its own: the build is chosen when the package is imported."""
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
    from rust_inference_b200.kernels import build, ops
    assert build.CHECKED and ops.checked_build() and build.library_path("elementwise").endswith("checked/libri_elementwise.so")
    model = make_model(pathlib.Path(tempfile.mkdtemp()), "A", std=0.08)
    toks = random_tokens(90, model.cfg["vocab_size"], seed=1)
    want = model.plain_logits(toks)
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=512)
        s = eng.alloc_slot()
        head = eng.step([s], [toks[:70]], "all").cpu()
        tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in toks[70:]])
        assert rel_err(torch.cat([head, tail]), want) <= (1e-4 if dtype == "float32" else 4e-2)
        eng.check_device_status()                       # ordinary work: nothing recorded
    assert ops.bounds_report() == []
    # a token id beyond the vocabulary: recorded, its row left zero, nothing read outside the table
    vocab = model.cfg["vocab_size"]
    table = torch.randn(vocab, 32, device="cuda")
    out = torch.full((3, 32), 7.0, device="cuda")
    ops.embed_gather(table, torch.tensor([1, vocab + 5, 2], dtype=torch.int32, device="cuda"), out)
    torch.cuda.synchronize()
    assert torch.equal(out[0], table[1]) and torch.equal(out[2], table[2]) and float(out[1].abs().max()) == 0.0
    rep = ops.bounds_report()
    assert rep == [("elementwise", "a token id outside the vocabulary", vocab + 5, vocab, 1)], rep
    assert ops.bounds_report() == []                    # read once, then cleared
    try:
        ops.embed_gather(table, torch.tensor([-1], dtype=torch.int32, device="cuda"), out[:1])
        eng.check_device_status()
    except ops.KernelError as e:
        assert "a token id outside the vocabulary (-1, limit" in str(e), e
    else:
        raise AssertionError("the engine's check did not speak")
    # a page-table entry beyond the pool: recorded, nothing written to the cache
    nh, nkv, hd = 2, 1, 16
    qkv = torch.randn(2, (nh + 2 * nkv) * hd, device="cuda")
    cos, sin = torch.ones(8, hd // 2, device="cuda"), torch.zeros(8, hd // 2, device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    n_pages = eng.cache.n_pages
    kc = torch.zeros(n_pages, nkv, 64, hd, device="cuda"); vc = torch.zeros_like(kc)
    table_bad = i32([[n_pages + 3], [0]])
    ops.rope_cache_write(qkv, cos, sin, i32([0, 1]), i32([0, 1]), i32([0, 1]), table_bad, kc, vc, n_heads=nh,
                         n_kv_heads=nkv, head_dim=hd, page_size=64, style=0, write_kv=True)
    torch.cuda.synchronize()
    rep = ops.bounds_report()
    assert rep == [("elementwise", "a page that does not exist", n_pages + 3, n_pages, 1)], rep
    assert float(kc[0, 0, 1].abs().max()) > 0 and float(kc[0, 0, 0].abs().max()) == 0.0   # the good token was stored, the bad one nowhere
    print("checked build ok")
""")


def test_the_checked_build_is_silent_on_ordinary_work_and_speaks_on_a_bad_index():
    env = dict(os.environ, RI_B200_CHECK_BOUNDS="1")
    proc = subprocess.run([sys.executable, "-c", SCRIPT.format(root=ROOT, tests=os.path.join(ROOT, "tests"))],
                          env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0 and "checked build ok" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-3000:]


def test_the_ordinary_build_has_no_checks():
    from rust_inference_b200.kernels import build, ops
    if build.CHECKED:
        pytest.skip("this process runs the checked build")
    ops.load("elementwise")
    with pytest.raises(ops.KernelError, match="not a checked build"):
        ops._limits = None
        ops.bounds_set_limits(10, 10, 10)
    ops._limits = None
    ops._limited.clear()
