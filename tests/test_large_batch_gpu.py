"""Decode steps of many sequences inside the engine: 80 sequences of unequal length step together, so
that sequences x kv heads exceed the number of SMs and the bf16 step takes the decode-attention kernel
that streams whole sequences through a TMA ring (no key split, no scratch), under a captured graph;
and generation over the same number of prompts with temperature sampling, with a vocabulary large
enough that a thread-block cluster samples each row.  Everything is compared with the plain
implementation (attention.rs:95-121, sampler.rs:72-106)."""
import pytest
import torch

from conftest import (TOL, assert_sampled_within_band, make_model, oracle_generate, random_tokens, rel_err,
                      top_k_agrees)

pytestmark = pytest.mark.gpu

N_SEQS = 80


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_eighty_sequences_decode_together(name, dtype, model_factory):
    from rust_inference_b200.engine.engine import Engine
    from rust_inference_b200.kernels import attention as attn
    model = model_factory(name, std=0.08)
    vocab = model.cfg["vocab_size"]
    n_steps = 6
    lens = [1 + (37 * i) % 150 for i in range(N_SEQS)]                 # 1 .. 150, unequal, some cross a page
    seqs = [random_tokens(n + n_steps, vocab, seed=500 + i) for i, n in enumerate(lens)]
    want = [model.plain_logits(s) for s in seqs]
    eng = Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=N_SEQS * 192)
    if dtype == "bfloat16":
        plan = attn.decode_plan(N_SEQS, model.cfg["num_key_value_heads"], eng.cache.page_table.shape[1] * 64, 64)
        assert plan == ("tma", 1) or attn._DECODE != "auto"          # unless the environment forces a kernel
    slots = [eng.alloc_slot() for _ in seqs]
    for g in range(0, N_SEQS, 16):                                      # prompts in unequal groups of 16
        got = eng.step(slots[g:g + 16], [s[:n] for s, n in zip(seqs[g:g + 16], lens[g:g + 16])], "last").cpu()
        for i in range(16):
            assert rel_err(got[i], want[g + i][lens[g + i] - 1]) <= TOL[dtype]
    worst = 0.0
    for step in range(n_steps):
        got = eng.step(slots, [[s[n + step]] for s, n in zip(seqs, lens)], "last").cpu()
        for i in range(N_SEQS):
            w = want[i][lens[i] + step]
            worst = max(worst, rel_err(got[i], w))
            assert top_k_agrees(got[i], w, 5, TOL[dtype]), (step, i)
        assert worst <= TOL[dtype], (step, worst)
    graph = eng.decode_graph(N_SEQS)
    assert graph.graph is not None and graph.eager_steps >= 3           # the last steps were replays
    eng.check_device_status()
    eng.cache.pager.audit()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_eighty_prompts_sampled_with_a_large_vocabulary(dtype, tmp_path):
    """Vocabulary 33,001: every row of logits is sampled by a cluster of eight thread blocks."""
    from rust_inference_b200 import Model, SamplerConfig
    model = make_model(tmp_path, "A", seed=9, std=0.08, overrides={"vocab_size": 33001, "num_hidden_layers": 1})
    prompts = [random_tokens(1 + (11 * i) % 23, 33001, seed=900 + i) for i in range(N_SEQS)]
    cfg = SamplerConfig.plain(temperature=0.8, seed=11)
    m = Model.load(model.folder, dtype=dtype, max_tokens_in_cache=N_SEQS * 64)
    from rust_inference_b200.kernels import ops
    ops.sample_cluster_any_rows(True)            # left to itself the library gives so many rows a block each
    try:
        got = m.generate(prompts, 5, cfg, stop_ids=())
    finally:
        ops.sample_cluster_any_rows(False)
    assert len(got) == N_SEQS and all(len(g.tokens) == 5 for g in got)
    for i in range(0, N_SEQS, 5 if dtype == "float32" else 9):          # a sample of the requests (the oracle is slow)
        if dtype == "float32":
            assert got[i].tokens == oracle_generate(model, prompts[i], 5, temperature=0.8, seed=11, stream=i), i
        else:
            assert_sampled_within_band(model, prompts[i], got[i].tokens, temperature=0.8, seed=11, stream=i, band=0.02)
    m.engine.check_device_status()
    m.engine.cache.pager.audit()
