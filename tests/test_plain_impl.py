"""The plain implementation checked against direct restatements of the reference's loops (no GPU)."""
import math

import pytest
import torch

import plain_impl
from conftest import TINY, make_model


def test_rmsnorm_is_the_reference_loop():
    x = torch.randn(3, 10)
    w = torch.randn(10)
    eps = 1e-5
    want = torch.empty_like(x)
    for r in range(3):                       # math.rs:237-256, literally
        ss = 0.0
        for i in range(10):
            ss += float(x[r, i]) ** 2
        scale = 1.0 / math.sqrt(ss / 10 + eps)
        for i in range(10):
            want[r, i] = float(x[r, i]) * scale * float(w[i])
    assert torch.allclose(plain_impl.rmsnorm(x, w, eps), want, atol=1e-6)


def test_silu_both_branches():
    x = torch.tensor([-30.0, -2.0, -0.0, 0.0, 0.5, 3.0, 40.0])
    want = torch.tensor([v / (1 + math.exp(-v)) if v >= 0 else v * math.exp(v) / (1 + math.exp(v)) for v in x.tolist()])
    assert torch.allclose(plain_impl.silu(x), want, atol=1e-7)
    assert torch.isfinite(plain_impl.silu(torch.tensor([-1e4, 1e4]))).all()


def test_rope_table_and_pairings():
    hd, base, n = 8, 10000.0, 5
    cos, sin = plain_impl.rope_table(hd, base, n)
    assert cos.shape == (n, hd // 2)
    for pos in (0, 3):
        for i in range(hd // 2):             # rope.rs:47-55
            theta = 1.0 / base ** ((2 * i) / hd)
            assert abs(cos[pos, i].item() - math.cos(pos * theta)) < 1e-6
            assert abs(sin[pos, i].item() - math.sin(pos * theta)) < 1e-6
    x = torch.randn(n, hd)
    inter = plain_impl.rope_apply(x, cos, sin, "interleaved")
    for i in range(hd // 2):                 # rope.rs:88-97
        assert torch.allclose(inter[:, 2 * i], x[:, 2 * i] * cos[:, i] - x[:, 2 * i + 1] * sin[:, i])
        assert torch.allclose(inter[:, 2 * i + 1], x[:, 2 * i] * sin[:, i] + x[:, 2 * i + 1] * cos[:, i])
    # the two pairings differ by a fixed permutation inside the head
    perm = torch.cat([torch.arange(0, hd, 2), torch.arange(1, hd, 2)])
    half = plain_impl.rope_apply(x[:, perm], cos, sin, "half")
    assert torch.allclose(half, inter[:, perm], atol=1e-6)
    # position 0 rotates nothing; norms are kept
    assert torch.allclose(inter[0], x[0]) and torch.allclose(inter.norm(dim=1), x.norm(dim=1), atol=1e-5)


def test_attention_is_the_reference_token_loop():
    torch.manual_seed(0)
    n, nh, nkv, hd, h = 6, 4, 2, 8, 16
    p = {"q_proj.weight": torch.randn(nh * hd, h) * 0.3, "k_proj.weight": torch.randn(nkv * hd, h) * 0.3,
         "v_proj.weight": torch.randn(nkv * hd, h) * 0.3, "o_proj.weight": torch.randn(h, nh * hd) * 0.3,
         "q_proj.bias": torch.randn(nh * hd) * 0.1, "k_proj.bias": torch.randn(nkv * hd) * 0.1,
         "v_proj.bias": torch.randn(nkv * hd) * 0.1}
    x = torch.randn(n, h)
    cos, sin = plain_impl.rope_table(hd, 10000.0, n)
    got, _ = plain_impl.attention(x, p, "", n_heads=nh, n_kv_heads=nkv, head_dim=hd, cos=cos, sin=sin,
                                  rope_style="interleaved")
    # attention.rs:54-124, one token at a time with a growing cache
    keys, vals, want = [], [], []
    n_rep = nh // nkv
    for pos in range(n):
        q = p["q_proj.weight"] @ x[pos] + p["q_proj.bias"]
        k = p["k_proj.weight"] @ x[pos] + p["k_proj.bias"]
        v = p["v_proj.weight"] @ x[pos] + p["v_proj.bias"]
        q = torch.cat([plain_impl.rope_apply(q[i * hd:(i + 1) * hd][None], cos[pos:pos + 1], sin[pos:pos + 1], "interleaved")[0] for i in range(nh)])
        k = torch.cat([plain_impl.rope_apply(k[i * hd:(i + 1) * hd][None], cos[pos:pos + 1], sin[pos:pos + 1], "interleaved")[0] for i in range(nkv)])
        keys.append(k)
        vals.append(v)
        out = torch.zeros(nh * hd)
        for hh in range(nh):
            kv = hh // n_rep
            scores = torch.tensor([float(q[hh * hd:(hh + 1) * hd] @ keys[j][kv * hd:(kv + 1) * hd]) / math.sqrt(hd)
                                   for j in range(pos + 1)])
            pr = plain_impl.softmax_rows(scores[None])[0]
            for j in range(pos + 1):
                out[hh * hd:(hh + 1) * hd] += pr[j] * vals[j][kv * hd:(kv + 1) * hd]
        want.append(p["o_proj.weight"] @ out)
    assert torch.allclose(got, torch.stack(want), atol=1e-5)


def test_window_and_shared_keys(tmp_path):
    m = make_model(tmp_path, "C", std=0.2, matrix_dtype=torch.float32)
    toks = list(range(1, 40))
    full = m.plain_logits(toks)
    # a schedule that names each layer once is the default
    assert torch.equal(full, m.plain_logits(toks, schedule=[(0, None), (1, None)]))
    # layer 1 reading layer 0's keys and values changes the result; running layer 0 twice as well
    assert not torch.allclose(full, m.plain_logits(toks, schedule=[(0, None), (1, 0)]))
    assert not torch.allclose(full, m.plain_logits(toks, schedule=[(0, None), (0, None), (1, None)]))
    # causality: logits at a position do not depend on later tokens
    assert torch.allclose(full[:10], m.plain_logits(toks[:10]), atol=1e-6)


def test_tied_head_uses_the_embedding(tmp_path):
    m = make_model(tmp_path, "A", matrix_dtype=torch.float32)
    assert "lm_head.weight" not in m.weights
    out = m.plain_logits([3, 4, 5])
    assert out.shape == (3, TINY["A"]["vocab_size"])


def test_sampling_functions():
    logits = torch.tensor([1.0, 3.0, 3.0, -1.0, 0.5])
    assert plain_impl.argmax_first(logits) == 1                                  # first maximum
    pen = plain_impl.repetition_penalty(logits, [3, 1, 1], penalty=2.0, window=64)
    assert pen.tolist() == [1.0, 0.75, 3.0, -2.0, 0.5]                           # repeats apply again
    assert plain_impl.repetition_penalty(logits, [0, 1, 3], 2.0, window=1).tolist() == [1.0, 3.0, 3.0, -2.0, 0.5]
    probs = torch.tensor([0.1, 0.4, 0.2, 0.2, 0.1])
    assert torch.allclose(plain_impl.top_k_filter(probs, 2), torch.tensor([0, 0.5, 0.25, 0.25, 0]))  # ties kept
    assert torch.allclose(plain_impl.top_p_filter(probs, 0.55), torch.tensor([0, 2 / 3, 1 / 3, 0, 0]))  # stable order
    assert torch.equal(plain_impl.top_p_filter(probs, 1.0), probs)
    assert plain_impl.draw(probs, 0.05) == 0 and plain_impl.draw(probs, 0.5) == 1 and plain_impl.draw(probs, 0.95) == 4
    assert plain_impl.draw(torch.tensor([0.3, 0.3]), 0.9) == 1                   # never reached: last index
    assert plain_impl.sample(logits, temperature=0.0, r=0.3) == 1
    assert plain_impl.sample(logits, temperature=0.0, r=0.3, penalty=2.0, recent=[1]) == 2   # penalty before greedy
    assert plain_impl.sample(logits, temperature=1.0, r=1e-6) == 0


def test_greedy_generate_stops_without_emitting(tmp_path):
    m = make_model(tmp_path, "C", std=0.2, matrix_dtype=torch.float32)
    out = plain_impl.greedy_generate(m.weights, m.cfg, [5, 6, 7], 6)
    assert len(out) == 6
    stop = out[2]
    cut = plain_impl.greedy_generate(m.weights, m.cfg, [5, 6, 7], 6, stop_ids=(stop,))
    assert cut == out[:out.index(stop)]


# ----------------------------------------------------------------------------------------
# A second statement of the same formulas: tests/golden/scalar_decoder.cpp (scalar loops, one token
# at a time, a cache).  Its logits on the tiny configurations are stored beside it.
# ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_implementation_agrees_with_the_scalar_program(name):
    import json
    import os
    import sys
    import numpy as np
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, golden)
    import make_golden
    with open(os.path.join(golden, f"{name}.json")) as f:
        meta = json.load(f)
    want = torch.from_numpy(np.fromfile(os.path.join(golden, f"{name}.logits.f32"), dtype=np.float32)
                            .reshape(meta["shape"]))
    cfg, w = make_golden.tiny_weights(name)
    assert make_golden.tokens_of(name, cfg.vocab_size) == meta["tokens"]
    weights = {k: torch.from_numpy(v) for k, v in w.items()}
    got = plain_impl.forward(weights, cfg.to_dict(), meta["tokens"])
    assert got.shape == want.shape
    err = ((got - want).abs().max() / want.abs().max()).item()
    assert err <= 2e-5, err                                 # two orders of summation in float32


def test_the_scalar_program_reproduces_its_stored_logits(tmp_path):
    """Where a C++ compiler is at hand, build the scalar program and run it again."""
    import json
    import os
    import shutil
    import sys
    import numpy as np
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, golden)
    import make_golden
    binary = make_golden.build(str(tmp_path))
    cfg, w = make_golden.tiny_weights("A")
    with open(os.path.join(golden, "A.json")) as f:
        meta = json.load(f)
    again = make_golden.run_scalar(binary, cfg, w, meta["tokens"], str(tmp_path))
    want = np.fromfile(os.path.join(golden, "A.logits.f32"), dtype=np.float32).reshape(meta["shape"])
    assert np.abs(again - want).max() <= 1e-6 * np.abs(want).max()


def test_storage_rounding_is_an_option_and_off_by_default(tmp_path):
    """`store_dtype` restates what keeping activations in bfloat16 between operations costs; without it
    nothing is rounded, and with float32 it is the identity."""
    m = make_model(tmp_path, "B", std=0.08)
    toks = list(range(3, 40))
    plain = plain_impl.forward(m.weights, m.cfg, toks)
    assert torch.equal(plain_impl.forward(m.weights, m.cfg, toks, store_dtype=torch.float32), plain)
    rounded = plain_impl.forward(m.weights, m.cfg, toks, store_dtype=torch.bfloat16)
    err = ((rounded - plain).abs().amax(dim=1) / plain.abs().amax(dim=1)).max().item()
    assert 1e-4 < err < 3e-2, err
