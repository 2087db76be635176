"""The benchmark model's own layer sizes (hidden 3584, 28 heads over 4 kv heads, head_dim 128,
intermediate 18944, vocabulary 152064, q/k/v biases) with one layer, in 32-bit and in bfloat16:
whole, with the last tokens decoded one by one, and in an unequal batch.  The plain implementation
runs on the GPU here (its tensor arithmetic is device-agnostic) with TF32 switched off."""
import json
import os

import pytest
import torch

from conftest import TOL, oracle_weights, random_tokens, rel_err

pytestmark = pytest.mark.gpu

SIZES = {
    "architectures": ["Qwen2ForCausalLM"], "hidden_size": 3584, "num_hidden_layers": 1,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944,
    "vocab_size": 152064, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True,
    "tie_word_embeddings": False, "max_position_embeddings": 8192,
}


@pytest.fixture(scope="module")
def big_model(tmp_path_factory):
    from rust_inference_b200 import config_from_dict, write_random_model
    folder = str(tmp_path_factory.mktemp("big") / "model")
    write_random_model(folder, config_from_dict(SIZES), seed=5, std=0.02, norm_std=0.2)
    weights = oracle_weights(folder, device="cuda")
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return folder, cfg, weights


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_sizes_in_every_cutting(dtype, big_model):
    import plain_impl
    from rust_inference_b200.engine.engine import Engine
    folder, cfg, weights = big_model
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        lens = [200, 1, 70, 620]               # the longest runs its SiLU-gate projection and its logits on pairs of SMs
        reqs = [random_tokens(n, cfg["vocab_size"], seed=n) for n in lens]
        want = [plain_impl.forward(weights, cfg, r).cpu() for r in reqs]
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=2048)
    tol = TOL[dtype]
    # whole and alone
    for r, w in zip(reqs, want):
        s = eng.alloc_slot()
        assert rel_err(eng.step([s], [r], "all"), w) <= tol
        eng.free_slot(s)
    # a prefix whole, then the last tokens one by one (decode kernels, CUDA graph)
    r, w = reqs[3], want[3]
    s = eng.alloc_slot()
    head = eng.step([s], [r[:-20]], "all").cpu()
    tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in r[-20:]])
    assert rel_err(torch.cat([head, tail]), w) <= tol
    eng.free_slot(s)
    # an unequal batch that starts together, then goes on by one token each
    cuts = [150, 1, 40, 560]
    slots = [eng.alloc_slot() for _ in reqs]
    got = eng.step(slots, [r[:c] for r, c in zip(reqs, cuts)], "all").cpu()
    off = 0
    for c, w in zip(cuts, want):
        assert rel_err(got[off:off + c], w[:c]) <= tol
        off += c
    live = [(s, r, c, w) for s, r, c, w in zip(slots, reqs, cuts, want) if c < len(r)]
    for step in range(6):
        live = [x for x in live if x[2] + step < len(x[1])]
        out = eng.step([x[0] for x in live], [[x[1][x[2] + step]] for x in live], "last").cpu()
        for i, x in enumerate(live):
            assert rel_err(out[i], x[3][x[2] + step]) <= tol
    eng.check_device_status()
