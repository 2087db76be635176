"""The benchmark model at its full depth: 28 layers of hidden 3584, 28 heads over 4 kv heads,
head_dim 128, intermediate 18944, vocabulary 152064, q/k/v biases, untied head, in true 32-bit and in
bfloat16, in every way of cutting the work, against the plain implementation (which computes
everything in float32 over the whole stack as the reference does, transformer.rs:63-98).

The weights are made here with torch on the GPU (values exactly representable in bfloat16, so both
precisions hold the same numbers; norm weights 1 + N(0, 0.2)) and handed to the model by name: the
plain implementation's weights do not pass through any part of the library.  One layer of these sizes
hides what 28 layers of sums, of atomic K-split additions and of 8,192-position rotary angles add up to."""
import pytest
import torch

import plain_impl
from conftest import TOL, random_tokens, rel_err, top_k_agrees

pytestmark = pytest.mark.gpu

SIZES = {
    "architectures": ["Qwen2ForCausalLM"], "hidden_size": 3584, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944,
    "vocab_size": 152064, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True,
    "tie_word_embeddings": False, "max_position_embeddings": 8192,
}
LENGTHS = [200, 1, 70, 620]


@pytest.fixture(scope="module")
def full_model():
    from rust_inference_b200 import config_from_dict
    from rust_inference_b200.config.registry import get_architecture
    from rust_inference_b200.engine.model import declared_tensors
    cfg = config_from_dict(SIZES)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    gen = torch.Generator(device="cuda").manual_seed(28)
    weights = {}
    for name, ts in declared_tensors(spec).items():
        t = torch.empty(ts.shape, dtype=torch.float32, device="cuda")
        if ts.init == "ones":
            t.normal_(0.0, 0.2, generator=gen).add_(1.0)
        else:
            t.normal_(0.0, 0.02, generator=gen)
        weights[name] = t.bfloat16().float() if ts.role == "matrix" else t
    reqs = [random_tokens(n, SIZES["vocab_size"], seed=1000 + n) for n in LENGTHS]
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False               # the oracle computes in true float32
    try:
        want = [plain_impl.forward(weights, SIZES, r).cpu() for r in reqs]
        # the same float32 arithmetic with everything that passes between two operations kept in
        # bfloat16: how far storage rounding alone moves the logits at this depth
        rounded = [plain_impl.forward(weights, SIZES, r, store_dtype=torch.bfloat16).cpu() for r in reqs]
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    storage_error = max(rel_err(a, b) for a, b in zip(rounded, want))
    del rounded
    yield spec, weights, reqs, want, storage_error
    weights.clear()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_twenty_eight_layers_in_every_cutting(dtype, full_model):
    from rust_inference_b200.engine.engine import Engine
    from rust_inference_b200.engine.model import DecoderModel
    spec, weights, reqs, want, storage_error = full_model
    model = DecoderModel(spec, dtype=torch.float32 if dtype == "float32" else torch.bfloat16, device="cuda")
    model.load(weights.items())
    eng = Engine(model, max_tokens=4096)
    # float32: the library's bound.  bfloat16: rounding noise adds up over the layers (it grows with the
    # square root of the depth: 0.011 at one layer of these sizes, 0.048 at 28), so the bound is taken
    # from the plain implementation itself: one and a half times what bfloat16 storage alone costs it
    # on these very requests.  A kernel fault shows as a multiple of that, and in float32 at 1e-4.
    tol = TOL[dtype] if dtype == "float32" else 1.5 * storage_error
    assert 0.02 < storage_error < 0.08
    observed = {}

    def check(got, w, what):
        err = rel_err(got, w)
        observed[what] = max(observed.get(what, 0.0), err)
        assert err <= tol, f"{dtype} {what}: {err:.3e}"
        for i in range(0, got.shape[0], max(1, got.shape[0] // 8)):
            assert top_k_agrees(got[i], w[i], 5, tol), f"{dtype} {what}: top-5 differs at row {i}"

    # 1. each request alone and whole
    for r, w in zip(reqs, want):
        s = eng.alloc_slot()
        check(eng.step([s], [r], "all").cpu(), w, "whole")
        eng.free_slot(s)
    # 2. a prefix whole, then the last 32 tokens one by one (decode kernels; the later steps replay a graph)
    for r, w in ((reqs[3], want[3]), (reqs[2], want[2])):
        s = eng.alloc_slot()
        head = eng.step([s], [r[:-32]], "all").cpu()
        tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in r[-32:]])
        check(torch.cat([head, tail]), w, "last 32 one by one")
        eng.free_slot(s)
    # 3. an unequal batch that starts together; shorter requests end earlier and free their slots;
    #    a second batch then takes the freed slots while the longest request of the first goes on
    cuts = [150, 1, 40, 560]
    slots = [eng.alloc_slot() for _ in reqs]
    got = eng.step(slots, [r[:c] for r, c in zip(reqs, cuts)], "all").cpu()
    off = 0
    for c, w in zip(cuts, want):
        check(got[off:off + c], w[:c], "unequal batch, prompts")
        off += c
    live = {i: cuts[i] for i in range(4) if cuts[i] < len(reqs[i])}
    for i in range(4):
        if i not in live:                                         # the one-token request ended with its prompt
            eng.free_slot(slots[i])
            slots[i] = None
    for _ in range(30):
        ids = sorted(live)
        out = eng.step([slots[i] for i in ids], [[reqs[i][live[i]]] for i in ids], "last").cpu()
        for row, i in enumerate(ids):
            check(out[row:row + 1], want[i][live[i]:live[i] + 1], "unequal batch, decode")
            live[i] += 1
            if live[i] == len(reqs[i]):
                del live[i]
                eng.free_slot(slots[i])
                slots[i] = None
    assert sorted(live) == [0, 3]                                 # requests 1 and 2 have ended and freed their slots
    second = {1: eng.alloc_slot(), 2: eng.alloc_slot()}           # the freed slots, taken again
    got = eng.step(list(second.values()), [reqs[2][:33], reqs[1]], "last").cpu()
    check(got[0:1], want[2][32:33], "second batch in reused slots")
    check(got[1:2], want[1][0:1], "second batch in reused slots")
    ids = [0, 3]
    for step in range(4):                                         # both batches decode together
        feed_slots = [slots[i] for i in ids] + [second[1]]
        feed = [[reqs[i][live[i]]] for i in ids] + [[reqs[2][33 + step]]]
        out = eng.step(feed_slots, feed, "last").cpu()
        for row, i in enumerate(ids):
            check(out[row:row + 1], want[i][live[i]:live[i] + 1], "both batches, decode")
            live[i] += 1
        check(out[2:3], want[2][33 + step:34 + step], "both batches, decode")
    eng.check_device_status()
    eng.cache.pager.audit()
    print(f"\nbound {tol:.2e} (bfloat16 storage alone moves the plain logits by {storage_error:.2e}); "
          f"observed worst relative errors, 28 layers, {dtype}: "
          + ", ".join(f"{k}: {v:.2e}" for k, v in observed.items()))
