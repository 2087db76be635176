"""The generation loop's decisions, with a scripted engine and sampler (no GPU)."""
import pytest

from rust_inference_b200.cache.pager import SlotPager
from rust_inference_b200.engine.generate import Generator


class FakeCache:
    def __init__(self, n_slots, n_pages, max_seq_len):
        self.pager = SlotPager(n_slots, n_pages, 64, max_seq_len)


class FakeEngine:
    """Keeps the real slot/page bookkeeping; a step only records what it was asked to run."""

    def __init__(self, n_slots=4, n_pages=16, max_seq_len=256):
        self.cache = FakeCache(n_slots, n_pages, max_seq_len)
        self.max_seq_len = max_seq_len
        self.calls = []

    def alloc_slot(self):
        return self.cache.pager.alloc_slot()

    def free_slot(self, slot):
        self.cache.pager.free_slot(slot)

    def step(self, slots, tokens, wants, borrow=False):
        pager = self.cache.pager
        pager.reserve_many([(s, pager.length(s) + len(t)) for s, t in zip(slots, tokens)])
        for s, t in zip(slots, tokens):
            pager.set_length(s, pager.length(s) + len(t))
        self.calls.append((list(slots), [list(t) for t in tokens]))
        return ("logits", len(slots))


class ScriptedSampler:
    """token = script(request index, how many it has drawn)."""

    def __init__(self, script):
        self.script = script
        self.seen = []

    def sample(self, logits, streams, counters, histories):
        self.seen.append((list(streams), list(counters)))
        return [self.script(s, c) for s, c in zip(streams, counters)]


def test_unequal_prompts_start_together_then_one_token_each():
    eng = FakeEngine()
    gen = Generator(eng, ScriptedSampler(lambda s, c: 100 + 10 * s + c))
    res = gen.generate([[1, 2, 3], [4] * 70, [7]], max_tokens=3)
    assert [r.tokens for r in res] == [[100, 101, 102], [110, 111, 112], [120, 121, 122]]
    assert all(r.finish_reason == "length" for r in res)
    assert [r.prompt_length for r in res] == [3, 70, 1]
    # first step: the whole prompts; then one token per sequence, the sampled one
    assert eng.calls[0][1] == [[1, 2, 3], [4] * 70, [7]]
    assert eng.calls[1][1] == [[100], [110], [120]]
    # no forward pass for the last sampled token: 1 prefill + 2 decode steps for 3 tokens
    assert len(eng.calls) == 3 and gen.steps == 3
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 4 and eng.cache.pager.free_page_count() == 16


def test_stop_token_ends_early_is_not_emitted_and_frees_the_slot():
    eng = FakeEngine()
    sampler = ScriptedSampler(lambda s, c: 9 if (s == 1 and c == 1) else 5)
    gen = Generator(eng, sampler, stop_ids=[9])
    res = gen.generate([[1], [2], [3]], max_tokens=4)
    assert res[1].tokens == [5] and res[1].finish_reason == "stop"
    assert res[0].tokens == [5, 5, 5, 5] and res[0].finish_reason == "length"
    # after sequence 1 stopped, the batch shrank to the two others
    assert [len(c[0]) for c in eng.calls] == [3, 3, 2, 2]
    assert sampler.seen[2][0] == [0, 2]
    eng.cache.pager.audit()


def test_stop_at_the_first_token():
    eng = FakeEngine()
    gen = Generator(eng, ScriptedSampler(lambda s, c: 9), stop_ids=[9])
    res = gen.generate([[1, 2]], max_tokens=8)
    assert res[0].tokens == [] and res[0].finish_reason == "stop" and len(eng.calls) == 1


def test_batches_follow_one_another_and_reuse_slots():
    eng = FakeEngine(n_slots=2, n_pages=16)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    res = gen.generate([[i + 1] * (i + 1) for i in range(5)], max_tokens=2)
    assert len(res) == 5 and all(r.tokens == [5, 5] for r in res)
    # 5 requests on 2 slots: batches of 2, 2, 1; each batch = prefill + 1 decode step
    assert [len(c[0]) for c in eng.calls] == [2, 2, 2, 2, 1, 1]
    used = {s for c in eng.calls for s in c[0]}
    assert used <= {0, 1}
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 2


def test_admission_counts_pages_for_the_whole_generation():
    # 4 pages of 64: a prompt of 60 with up to 10 more needs 2 pages, so only 2 requests fit at once
    eng = FakeEngine(n_slots=4, n_pages=4)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    res = gen.generate([[1] * 60] * 3, max_tokens=10)
    assert all(len(r.tokens) == 10 for r in res)
    assert len(eng.calls[0][0]) == 2
    eng.cache.pager.audit()


def test_a_request_that_cannot_fit_is_an_error():
    eng = FakeEngine(n_slots=2, n_pages=1)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    with pytest.raises(RuntimeError, match="does not fit"):
        gen.generate([[1] * 100], max_tokens=4)
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 2


def test_max_seq_len_ends_with_length():
    eng = FakeEngine(n_slots=1, n_pages=8, max_seq_len=70)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    res = gen.generate([[1] * 68], max_tokens=50)
    # positions 68 and 69 can still be fed; the token sampled after position 69 has nowhere to go
    assert len(res[0].tokens) == 3 and res[0].finish_reason == "length"
    assert eng.cache.pager.free_slot_count() == 1
    with pytest.raises(ValueError, match="exceeds max_seq_len"):
        gen.generate([[1] * 71], max_tokens=1)


def test_edge_cases():
    eng = FakeEngine()
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    with pytest.raises(ValueError, match="empty prompt"):
        gen.generate([[1], []], max_tokens=2)
    res = gen.generate([[1, 2]], max_tokens=0)
    assert res[0].tokens == [] and res[0].finish_reason == "length" and eng.calls == []
    assert gen.generate([], max_tokens=3) == []


def test_max_batch_limits_a_wave():
    eng = FakeEngine(n_slots=4)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5), max_batch=1)
    gen.generate([[1], [2], [3]], max_tokens=1)
    assert [len(c[0]) for c in eng.calls] == [1, 1, 1]


def test_slots_are_freed_when_a_step_raises():
    class Boom(FakeEngine):
        def step(self, *a, **k):
            if len(self.calls) == 1:
                raise RuntimeError("boom")
            return super().step(*a, **k)

    eng = Boom()
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    with pytest.raises(RuntimeError, match="boom"):
        gen.generate([[1], [2]], max_tokens=5)
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 4


def test_history_reaches_the_sampler_when_the_penalty_is_on():
    from rust_inference_b200 import SamplerConfig

    class HistSampler(ScriptedSampler):
        params = SamplerConfig(repetition_penalty=1.3)

        def sample(self, logits, streams, counters, histories):
            self.hist = [list(h) for h in histories]
            return super().sample(logits, streams, counters, histories)

    eng = FakeEngine()
    s = HistSampler(lambda st, c: 50 + c)
    Generator(eng, s).generate([[1, 2, 3]], max_tokens=3)
    assert s.hist == [[1, 2, 3, 50, 51]]            # prompt and generated tokens (model.rs:357, :364, :440)
