"""The two tiny workloads as they are stated for this library's benchmark description.

Configuration 1 (conftest.TINY["C"]: 2 layers, hidden 64, 8 heads over 2 kv heads, head_dim 8, tied):
a batch of 3 prompts of 5, 11 and 17 ids (seed 1), then 8 greedy decode steps, logits checked at every
position; and the resulting sequences replayed whole, with the last tokens one by one, and as a batch.
Configuration 2 (TINY["D"]: 3 layers, hidden 144, 6 heads over 3 kv heads, head_dim 24, biases, untied):
a batch of 4 prompts of 1, 7, 30 and 64 ids (seed 3), then 16 steps at temperature 0.7 with sampler
seed 4, in three ways of cutting the work: every prompt whole and alone, token by token, and all four
as one unequal batch; the sampled tokens must be those the plain implementation samples when it is fed
the same uniform numbers (the loop of model.rs:361-442 with sampler.rs:72-106).
Head sizes 8 and 24 run on the generic kernels in both precisions."""
import pytest
import torch

import plain_impl
from conftest import TOL, assert_sampled_within_band, oracle_generate, random_tokens, rel_err
from replay_util import batches, last_decoded, run_trace, whole, worst_error

pytestmark = pytest.mark.gpu


def _engine(model, dtype, **kw):
    from rust_inference_b200.engine.engine import Engine
    kw.setdefault("max_tokens", 1024)
    return Engine.from_pretrained(model.folder, dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_configuration_one_three_prompts_then_eight_greedy_steps(dtype, model_factory, tmp_path):
    model = model_factory("C", std=0.1)
    vocab = model.cfg["vocab_size"]
    prompts = [random_tokens(n, vocab, seed=1 + i) for i, n in enumerate((5, 11, 17))]
    eng = _engine(model, dtype)
    slots = [eng.alloc_slot() for _ in prompts]
    got = [list(eng.step(slots, prompts, "all").cpu().split([len(p) for p in prompts]))]   # logits at every prompt position
    rows = [[r] for r in got[0]]
    seqs = [list(p) for p in prompts]
    for _ in range(8):
        feed = [[int(r[-1][-1].argmax())] for r in rows]             # greedy on the engine's own logits
        for s, f in zip(seqs, feed):
            s.append(f[0])
        out = eng.step(slots, feed, "last").cpu()
        for r, o in zip(rows, out):
            r.append(o[None])
    for s, r in zip(seqs, rows):
        want = model.plain_logits(s)
        assert rel_err(torch.cat(r), want) <= TOL[dtype]             # every position, prompt and decoded
    if dtype == "float32":
        for p, s in zip(prompts, seqs):
            assert s[len(p):] == plain_impl.greedy_generate(model.weights, model.cfg, p, 8)
    # the same sequences through the replay program, cut three ways
    reqs = {f"p{i}": s for i, s in enumerate(seqs)}
    plain = {rid: model.plain_logits(s) for rid, s in reqs.items()}
    for mode, trace in {"whole": whole(reqs), "last8": last_decoded(reqs, 8),
                        "batch": batches([reqs, reqs], prompt_frac=0.4)}.items():
        out = run_trace(model.folder, dtype, trace, str(tmp_path / mode))
        err, step, rid, pos = worst_error(trace, out, plain)
        assert err <= TOL[dtype], f"{dtype} {mode}: rel err {err:.3e} at step {step}, {rid}, position {pos}"


def _token_by_token(eng, prompt, n_new, cfg, stream):
    """A sequence fed one token per step from its first token on, then sampled with the product's sampler."""
    from rust_inference_b200.sampling.sampler import Sampler
    sampler = Sampler(cfg, eng.device)
    s = eng.alloc_slot()
    for t in prompt[:-1]:
        eng.step([s], [[t]], "none")
    feed, out = prompt[-1], []
    for i in range(n_new):
        logits = eng.step([s], [[feed]], "last")
        feed = int(sampler.sample(logits, [stream], [i]).cpu()[0])
        out.append(feed)
    eng.free_slot(s)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_configuration_two_sixteen_steps_at_temperature_in_three_cuttings(dtype, model_factory):
    from rust_inference_b200 import Model, SamplerConfig
    model = model_factory("D", std=0.1)
    vocab = model.cfg["vocab_size"]
    prompts = [random_tokens(n, vocab, seed=3 + i) for i, n in enumerate((1, 7, 30, 64))]
    cfg = SamplerConfig.plain(temperature=0.7, seed=4)
    m = Model.load(model.folder, dtype=dtype, max_tokens_in_cache=1024)
    runs = {
        "mixed batch": [(i, r.tokens) for i, r in enumerate(m.generate(prompts, 16, cfg, stop_ids=()))],
        "whole and alone": [(0, m.generate([p], 16, cfg, stop_ids=())[0].tokens) for p in prompts],
        "token by token": [(i, _token_by_token(m.engine, p, 16, cfg, i)) for i, p in enumerate(prompts)],
    }
    for mode, got in runs.items():
        for p, (stream, tokens) in zip(prompts, got):
            assert len(tokens) == 16
            if dtype == "float32":
                want = oracle_generate(model, p, 16, temperature=0.7, seed=4, stream=stream)
                assert tokens == want, f"{mode}, prompt of {len(p)}"
            else:
                assert_sampled_within_band(model, p, tokens, temperature=0.7, seed=4, stream=stream, band=0.02)
    m.engine.cache.pager.audit()
    m.engine.check_device_status()
