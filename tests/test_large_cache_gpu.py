"""A cache so large that element offsets in one layer's keys exceed 2^31: the pages a sequence
gets lie at the far end of the pool, so every kernel that touches the cache (rotary write, prefill and
decode attention, in both precisions) has to compute its addresses in 64 bits."""
import pytest
import torch

from conftest import TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_pages_beyond_two_to_the_31_elements(dtype, tmp_path):
    from conftest import make_model
    from rust_inference_b200.engine.engine import Engine
    m = make_model(tmp_path, "A", seed=21, overrides={"num_hidden_layers": 1})
    per_page = 64 * m.cfg["num_key_value_heads"] * m.cfg["head_dim"]            # elements of one page in one layer
    n_pages = (1 << 31) // per_page + 6000
    eng = Engine.from_pretrained(m.folder, dtype=dtype, max_tokens=n_pages * 64, max_seq_len=1024, n_slots=4)
    pager = eng.cache.pager
    assert pager.n_pages == n_pages
    pager.prefer_high_pages()                        # hand out the highest page numbers first
    reqs = [random_tokens(n, m.cfg["vocab_size"], seed=n) for n in (300, 90)]
    want = [m.plain_logits(r) for r in reqs]
    tol = TOL[dtype]
    # whole, then the last tokens one by one
    s = eng.alloc_slot()
    head = eng.step([s], [reqs[0][:-6]], "all").cpu()
    assert min(pager.pages(s)) * per_page >= 1 << 31
    tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in reqs[0][-6:]])
    assert rel_err(torch.cat([head, tail]), want[0]) <= tol
    # an unequal batch in the pages next to them
    slots = [eng.alloc_slot() for _ in reqs]
    got = eng.step(slots, [r[:-2] for r in reqs], "all").cpu()
    off = 0
    for r, w in zip(reqs, want):
        assert rel_err(got[off:off + len(r) - 2], w[:len(r) - 2]) <= tol
        off += len(r) - 2
    for k in (2, 1):
        out = eng.step(slots, [[r[-k]] for r in reqs], "last").cpu()
        for i, w in enumerate(want):
            assert rel_err(out[i], w[len(reqs[i]) - k]) <= tol
    assert all(min(pager.pages(x)) * per_page >= 1 << 31 for x in slots)
    eng.check_device_status()
    for x in slots + [s]:
        eng.free_slot(x)
    pager.audit()
