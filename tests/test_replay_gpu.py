"""Trace replay through bin/trace_run, compared with the plain implementation: every request
alone and whole; with the last 32 tokens decoded one by one; in batches of unequal lengths
whose shorter requests end earlier, one batch after another so that slots are used again."""
import pytest
import torch

from conftest import TOL, random_tokens
from replay_util import batches, last_decoded, run_trace, top_k_disagreements, whole, worst_error

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 40, 97, 300, 64, 65], "B": [1, 33, 128, 211, 70, 450]}


def _requests(model, name):
    vocab = model.cfg["vocab_size"]
    return {f"r{i}": random_tokens(n, vocab, seed=10 * i + len(name)) for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_modes(name, dtype, model_factory, tmp_path):
    model = model_factory(name, std=0.08)
    reqs = _requests(model, name)
    plain = {rid: model.plain_logits(toks) for rid, toks in reqs.items()}
    long_reqs = {rid: t for rid, t in reqs.items() if len(t) > 32}
    ids = list(reqs)
    groups = [{r: reqs[r] for r in ids[:4]}, {r: reqs[r] for r in ids[4:]}, {r: reqs[r] for r in ids[1:5]}]
    traces = {"whole": whole(reqs), "last32": last_decoded(long_reqs, 32), "batches": batches(groups)}
    for mode, trace in traces.items():
        out = run_trace(model.folder, dtype, trace, str(tmp_path / f"{mode}"))
        err, step, rid, pos = worst_error(trace, out, plain)
        assert err <= TOL[dtype], (f"{name} {dtype} {mode}: rel err {err:.3e} at step {step}, request {rid}, "
                                   f"position {pos} (of {len(reqs[rid]) if rid else '?'})")
        assert top_k_disagreements(trace, out, plain, 5, TOL[dtype]) == [], f"{name} {dtype} {mode}: top-5"


@pytest.mark.parametrize("name", ["C", "D"])
def test_replay_small_heads(name, model_factory, tmp_path):
    """head_dim 8 and 24: both dtypes run on the generic kernels."""
    model = model_factory(name, std=0.1)
    vocab = model.cfg["vocab_size"]
    lens = [5, 11, 17] if name == "C" else [1, 7, 30, 64]
    reqs = {f"q{i}": random_tokens(n + 20, vocab, seed=i + 1) for i, n in enumerate(lens)}
    plain = {rid: model.plain_logits(toks) for rid, toks in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        trace = batches([reqs], prompt_frac=0.6)
        out = run_trace(model.folder, dtype, trace, str(tmp_path / dtype))
        err, step, rid, pos = worst_error(trace, out, plain)
        assert err <= TOL[dtype], f"{name} {dtype}: rel err {err:.3e} at step {step}, {rid}, position {pos}"


def test_replay_protocol(model_factory, tmp_path):
    """Nothing wanted writes no file; a request may be continued by several tokens; the process
    ends with 0 when its input ends."""
    from replay_util import Trace
    model = model_factory("A", std=0.08)
    toks = random_tokens(100, model.cfg["vocab_size"], seed=5)
    plain = {"x": model.plain_logits(toks)}
    t = Trace()
    t.add([("x", toks[:30], [], 0)])                       # nothing wanted
    t.add([("x", toks[30:75], [0, 44], 30)])               # a continuation of 45 tokens
    t.add([("x", toks[75:], range(25), 75)], end=["x"])
    out = run_trace(model.folder, "float32", t, str(tmp_path / "o"), max_tokens=128)
    assert sorted(out) == [1, 2]
    err, *_ = worst_error(t, out, plain)
    assert err <= TOL["float32"]
