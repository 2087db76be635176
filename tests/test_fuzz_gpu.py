"""Random schedules against the plain implementation: sequences that start, go on by one or by several
tokens, pause, end and give their slots to others, in random order and grouping; decode steps fed from
the host and from the device, the same group several times in a row (a captured step then moves its own
arrays on) and other groups in between; and random generation calls (batch limits, stop ids, lengths)
on one model, so that captured steps are reused across calls.  Every row of logits and every generated
token is checked; seeds are fixed, so a failure names its schedule."""
import os
import random

import pytest
import torch

import plain_impl
from conftest import TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu
SEEDS = list(range(int(os.environ.get("RI_TEST_FUZZ_SEEDS", "3"))))        # more seeds for a longer soak


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", SEEDS)
def test_random_schedules_of_steps(seed, dtype, model_factory):
    from rust_inference_b200.engine.engine import Engine
    name = "AB"[seed % 2]
    model = model_factory(name, std=0.08)
    vocab = model.cfg["vocab_size"]
    rng = random.Random(1000 + seed)
    eng = Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=6 * 192, n_slots=6)
    tol = TOL[dtype]
    pool = []                                            # requests not started yet: (tokens, plain logits)
    for i in range(14):
        toks = random_tokens(rng.randint(2, 150), vocab, seed=50 * seed + i)
        pool.append((toks, model.plain_logits(toks)))
    live = {}                                            # slot -> [tokens, plain logits, position]
    checked = 0

    def check(got, slot, pos, count):
        nonlocal checked
        assert rel_err(got, live[slot][1][pos:pos + count]) <= tol, (seed, dtype, slot, pos, count)
        checked += count

    def finish(slot):
        if live[slot][2] == len(live[slot][0]):
            eng.free_slot(slot)
            del live[slot]

    last_group = None
    for _ in range(120):
        op = rng.random()
        if (op < 0.25 or not live) and pool and len(live) < 6:
            # some requests start together with prompts of unequal length (whole, or a first part)
            k = min(rng.randint(1, 3), len(pool), 6 - len(live))
            new = []
            for _ in range(k):
                toks, want = pool.pop()
                slot = eng.alloc_slot()
                live[slot] = [toks, want, 0]
                new.append(slot)
            cuts = [rng.randint(1, len(live[s][0])) for s in new]
            got = eng.step(new, [live[s][0][:c] for s, c in zip(new, cuts)], "all").cpu()
            off = 0
            for s, c in zip(new, cuts):
                check(got[off:off + c], s, 0, c)
                off += c
                live[s][2] = c
                finish(s)
            last_group = None
        elif op < 0.4 and live:
            # a continuation by several tokens for one or two sequences
            group = rng.sample(sorted(live), min(len(live), rng.randint(1, 2)))
            counts = [min(rng.randint(2, 40), len(live[s][0]) - live[s][2]) for s in group]
            got = eng.step(group, [live[s][0][live[s][2]:live[s][2] + c] for s, c in zip(group, counts)], "all").cpu()
            off = 0
            for s, c in zip(group, counts):
                check(got[off:off + c], s, live[s][2], c)
                off += c
                live[s][2] += c
                finish(s)
            last_group = None
        elif live:
            # one token each for a group: the same group as before (its captured step holds its arrays),
            # or another one; fed from the host or from a device tensor
            if last_group and all(s in live for s in last_group) and rng.random() < 0.6:
                group = last_group
            else:
                group = rng.sample(sorted(live), rng.randint(1, len(live)))
            feed = [live[s][0][live[s][2]] for s in group]
            if rng.random() < 0.5:
                got = eng.step(group, [[t] for t in feed], "last").cpu()
            else:
                got = eng.step_from_device(group, torch.tensor(feed, dtype=torch.int32, device="cuda")).cpu()
            for i, s in enumerate(group):
                check(got[i:i + 1], s, live[s][2], 1)
                live[s][2] += 1
            last_group = list(group)
            for s in group:
                finish(s)
    assert checked > 400
    eng.check_device_status()
    eng.cache.pager.audit()


@pytest.mark.parametrize("seed", SEEDS[:max(2, len(SEEDS) // 2)])
def test_random_generation_calls_on_one_model(seed, model_factory):
    from rust_inference_b200 import Model, SamplerConfig
    model = model_factory("A", std=0.08)
    vocab = model.cfg["vocab_size"]
    rng = random.Random(77 + seed)
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=8 * 128, n_slots=5)
    greedy = SamplerConfig.plain(0.0)
    for call in range(6):
        n = rng.randint(1, 9)
        prompts = [random_tokens(rng.randint(1, 40), vocab, seed=1000 * seed + 20 * call + i) for i in range(n)]
        max_tokens = rng.randint(1, 12)
        free = [plain_impl.greedy_generate(model.weights, model.cfg, p, max_tokens) for p in prompts]
        # stop ids taken from what the model does generate, so that some sequences stop early
        stops = tuple({seq[rng.randrange(len(seq))] for seq in free if rng.random() < 0.5})
        want = [plain_impl.greedy_generate(model.weights, model.cfg, p, max_tokens, stop_ids=stops) for p in prompts]
        got = m.generate(prompts, max_tokens, greedy, stop_ids=stops, max_batch=rng.choice([None, 1, 2, 4]))
        assert [g.tokens for g in got] == want, (seed, call, stops)
        for g, w, f in zip(got, want, free):
            assert g.finish_reason == ("length" if len(w) == max_tokens else "stop")
        m.engine.cache.pager.audit()
        assert m.engine.cache.pager.free_slot_count() == 5
    m.engine.check_device_status()
