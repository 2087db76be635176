"""The generation loop's decisions, with a scripted engine and sampler (no GPU).

Every test runs over both loops: the plain one (step, sample, read, decide) and the one every real
engine takes, which looks one step ahead (`Generator._run_batch_ahead`): there the engine can feed a
step from the device, the sampler writes into a host buffer and the loop waits for a mark.  The
stand-ins below are numpy arrays and marks that do nothing."""
import numpy as np
import pytest

from rust_inference_b200.cache.pager import SlotPager
from rust_inference_b200.engine.generate import Generator as _Generator


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


class AheadEngine(FakeEngine):
    """The same books, plus what lets the loop look ahead: a step fed from a 'device' array."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.token_buffers = {}
        self.fed_in_place = 0

    def can_feed_from_device(self):
        return True

    def decode_token_buffer(self, n):
        return self.token_buffers.setdefault(n, np.zeros(n, dtype=np.int32))

    def step_from_device(self, slots, tokens_dev):
        assert len(tokens_dev) == len(slots)
        if tokens_dev is self.token_buffers.get(len(slots)):
            self.fed_in_place += 1
        return self.step(slots, [[int(t)] for t in tokens_dev], "last")


class InStepEngine(AheadEngine):
    """An engine whose decode steps hold the sampler: one call runs the step and samples, and hands back
    the tokens on the 'device' (the buffer the next step reads) and in 'pinned host' memory."""

    def __init__(self, script, *a, **k):
        super().__init__(*a, **k)
        self.script = script
        self.sampled_in_step = []
        self.host_ring = {}

    def can_sample_in_step(self, params):
        return not params.uses_history

    def decode_token_buffer(self, n, sampler=None):
        return self.token_buffers.setdefault(n, np.zeros(n, dtype=np.int32))

    def step_and_sample_from_device(self, slots, tokens_dev, params, streams, counters):
        self.step_from_device(slots, tokens_dev)
        self.sampled_in_step.append((list(streams), list(counters)))
        toks = [self.script(s, c) for s, c in zip(streams, counters)]
        dev = self.decode_token_buffer(len(slots))
        dev[:] = toks
        ring = self.host_ring.setdefault(len(slots), [np.zeros(len(slots), dtype=np.int32) for _ in range(4)])
        host = ring[len(self.sampled_in_step) % 4]
        host[:] = toks
        return dev, host


class FakeMark:
    waited = 0

    def synchronize(self):
        FakeMark.waited += 1


class FakeLoopDevice:
    def host_buffer(self, n):
        return np.full(n, -1, dtype=np.int32)

    def mark(self):
        return FakeMark()

    def rows(self, tokens, keep):
        return np.asarray(tokens)[list(keep)].copy()


class ScriptedSampler:
    """token = script(request index, how many it has drawn)."""

    def __init__(self, script):
        self.script = script
        self.seen = []

    def sample(self, logits, streams, counters, histories=None, out=None, mirror=None, newest=None):
        self.seen.append((list(streams), list(counters)))
        toks = [self.script(s, c) for s, c in zip(streams, counters)]
        if out is None and mirror is None:
            return toks                                   # the plain loop reads what is returned
        dev = out if out is not None else np.zeros(len(toks), dtype=np.int32)
        dev[:] = toks
        if mirror is not None:
            mirror[:] = toks
        return dev


@pytest.fixture(params=["plain", "ahead", "in_step"])
def loop(request):
    """plain: step, sample, read, decide.  ahead: one step of lookahead, the sampler called after each
    step.  in_step: lookahead with the sampler inside the engine's decode step."""
    return request.param


ENGINES = {"plain": FakeEngine, "ahead": AheadEngine}


def make_engine(loop, *a, **k):
    if loop == "in_step":
        return InStepEngine(None, *a, **k)          # the script comes with the sampler (see Generator below)
    return ENGINES[loop](*a, **k)


def Generator(engine, sampler, **k):
    if isinstance(engine, InStepEngine):
        from rust_inference_b200 import SamplerConfig
        engine.script = sampler.script
        if not hasattr(sampler, "params"):
            sampler.params = SamplerConfig.plain(0.0)
    return _Generator(engine, sampler, device=FakeLoopDevice(), **k)


def test_unequal_prompts_start_together_then_one_token_each(loop):
    eng = make_engine(loop)
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


def test_stop_token_ends_early_is_not_emitted_and_frees_the_slot(loop):
    eng = make_engine(loop)
    sampler = ScriptedSampler(lambda s, c: 9 if (s == 1 and c == 1) else 5)
    gen = Generator(eng, sampler, stop_ids=[9])
    res = gen.generate([[1], [2], [3]], max_tokens=4)
    assert res[1].tokens == [5] and res[1].finish_reason == "stop"
    assert res[0].tokens == [5, 5, 5, 5] and res[0].finish_reason == "length"
    if loop == "plain":
        # after sequence 1 stopped, the batch shrank to the two others
        assert [len(c[0]) for c in eng.calls] == [3, 3, 2, 2]
        assert sampler.seen[2][0] == [0, 2]
    else:
        # one step ahead: when the stop token is read, the step that feeds it already runs (three
        # rows); its row is dropped and the stop token is fed no further
        assert [len(c[0]) for c in eng.calls] == [3, 3, 3, 2]
        assert eng.calls[2][1] == [[5], [9], [5]] and eng.calls[3][1] == [[5], [5]]
        # who was sampled: after the prompts' step the sampler object; in the in_step loop every later
        # sample happens inside the engine's step
        seen = [x[0] for x in sampler.seen] + [x[0] for x in getattr(eng, "sampled_in_step", [])]
        assert seen == [[0, 1, 2], [0, 1, 2], [0, 1, 2], [0, 2]]
    assert res[2].tokens == [5, 5, 5, 5]
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 4


def test_stop_at_the_first_token(loop):
    eng = make_engine(loop)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 9), stop_ids=[9])
    res = gen.generate([[1, 2]], max_tokens=8)
    assert res[0].tokens == [] and res[0].finish_reason == "stop"
    # the loop that looks ahead has fed the stop token once before it read it
    assert len(eng.calls) == (1 if loop == "plain" else 2)
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 4


def test_batches_follow_one_another_and_reuse_slots(loop):
    eng = make_engine(loop, n_slots=2, n_pages=16)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    res = gen.generate([[i + 1] * (i + 1) for i in range(5)], max_tokens=2)
    assert len(res) == 5 and all(r.tokens == [5, 5] for r in res)
    # 5 requests on 2 slots: batches of 2, 2, 1; each batch = prefill + 1 decode step
    assert [len(c[0]) for c in eng.calls] == [2, 2, 2, 2, 1, 1]
    used = {s for c in eng.calls for s in c[0]}
    assert used <= {0, 1}
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 2


def test_admission_counts_pages_for_the_whole_generation(loop):
    # 4 pages of 64: a prompt of 60 with up to 10 more needs 2 pages, so only 2 requests fit at once
    eng = make_engine(loop, n_slots=4, n_pages=4)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    res = gen.generate([[1] * 60] * 3, max_tokens=10)
    assert all(len(r.tokens) == 10 for r in res)
    assert len(eng.calls[0][0]) == 2
    eng.cache.pager.audit()


def test_a_request_that_cannot_fit_is_an_error(loop):
    eng = make_engine(loop, n_slots=2, n_pages=1)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    with pytest.raises(RuntimeError, match="does not fit"):
        gen.generate([[1] * 100], max_tokens=4)
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 2


def test_max_seq_len_ends_with_length(loop):
    eng = make_engine(loop, n_slots=1, n_pages=8, max_seq_len=70)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    res = gen.generate([[1] * 68], max_tokens=50)
    # positions 68 and 69 can still be fed; the token sampled after position 69 has nowhere to go
    assert len(res[0].tokens) == 3 and res[0].finish_reason == "length"
    assert eng.cache.pager.free_slot_count() == 1
    with pytest.raises(ValueError, match="exceeds max_seq_len"):
        gen.generate([[1] * 71], max_tokens=1)


def test_edge_cases(loop):
    eng = make_engine(loop)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5))
    with pytest.raises(ValueError, match="empty prompt"):
        gen.generate([[1], []], max_tokens=2)
    res = gen.generate([[1, 2]], max_tokens=0)
    assert res[0].tokens == [] and res[0].finish_reason == "length" and eng.calls == []
    assert gen.generate([], max_tokens=3) == []


def test_max_batch_limits_a_wave(loop):
    eng = make_engine(loop, n_slots=4)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 5), max_batch=1)
    gen.generate([[1], [2], [3]], max_tokens=1)
    assert [len(c[0]) for c in eng.calls] == [1, 1, 1]


def test_slots_are_freed_when_a_step_raises(loop):
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


def test_history_reaches_the_sampler_when_the_penalty_is_on(loop):
    from rust_inference_b200 import SamplerConfig

    class HistSampler(ScriptedSampler):
        params = SamplerConfig(repetition_penalty=1.3)

        def sample(self, logits, streams, counters, histories=None, out=None, mirror=None, newest=None):
            self.hist = [list(h) for h in histories]
            self.newest = None if newest is None else [int(t) for t in newest]
            return super().sample(logits, streams, counters, histories, out=out, mirror=mirror, newest=newest)

    eng = make_engine(loop)
    s = HistSampler(lambda st, c: 50 + c)
    Generator(eng, s).generate([[1, 2, 3]], max_tokens=3)
    if loop == "plain":
        assert s.hist == [[1, 2, 3, 50, 51]]        # prompt and generated tokens (model.rs:357, :364, :440)
    else:
        # the newest token has not reached the host when the next one is sampled: the sampler is given
        # it on the device, and the host's history holds the ones before
        assert s.hist == [[1, 2, 3, 50]] and s.newest == [51]


# ----------------------------------------------------------------------------------------
# Cases of the loop that looks ahead
# ----------------------------------------------------------------------------------------
def test_two_sequences_stop_in_the_same_step(loop):
    eng = make_engine(loop)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 9 if (s in (0, 2) and c == 2) else 40 + s), stop_ids=[9])
    res = gen.generate([[1], [2, 2], [3, 3, 3], [4]], max_tokens=5)
    assert [r.tokens for r in res] == [[40, 40], [41] * 5, [42, 42], [43] * 5]
    assert [r.finish_reason for r in res] == ["stop", "length", "stop", "length"]
    sizes = [len(c[0]) for c in eng.calls]
    assert sizes == ([4, 4, 4, 2, 2] if loop == "plain" else [4, 4, 4, 4, 2])
    assert 9 not in [t for c in eng.calls[-1:] for toks in c[1] for t in toks]
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 4 and eng.cache.pager.free_page_count() == 16


def test_every_sequence_stops_while_a_step_is_in_flight(loop):
    eng = make_engine(loop, n_slots=2)
    gen = Generator(eng, ScriptedSampler(lambda s, c: 9 if c == 1 else 7), stop_ids=[9])
    res = gen.generate([[1], [2], [3]], max_tokens=6)            # two batches on two slots
    assert [r.tokens for r in res] == [[7], [7], [7]] and all(r.finish_reason == "stop" for r in res)
    sizes = [len(c[0]) for c in eng.calls]
    # plain: prefill + one decode step per batch; ahead: one more step per batch, run for nothing
    assert sizes == ([2, 2, 1, 1] if loop == "plain" else [2, 2, 2, 1, 1, 1])
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 2 and eng.cache.pager.free_page_count() == 16


def test_one_ends_at_max_seq_len_a_step_before_another_stops(loop):
    eng = make_engine(loop, n_slots=2, n_pages=8, max_seq_len=70)
    # request 0 (prompt 67) can be fed at positions 67, 68, 69: it ends by length with its 4th token;
    # request 1 samples a stop token as its 5th
    gen = Generator(eng, ScriptedSampler(lambda s, c: 9 if (s == 1 and c == 4) else 20 + s), stop_ids=[9])
    res = gen.generate([[1] * 67, [2] * 3], max_tokens=30)
    assert res[0].tokens == [20] * 4 and res[0].finish_reason == "length"
    assert res[1].tokens == [21] * 4 and res[1].finish_reason == "stop"
    sizes = [len(c[0]) for c in eng.calls]
    # the sequence that ends by length is never stepped beyond its last position in either loop
    assert sizes == ([2, 2, 2, 2, 1] if loop == "plain" else [2, 2, 2, 2, 1, 1])
    assert max(len(t) for c in eng.calls[1:] for t in c[1]) == 1
    eng.cache.pager.audit()
    assert eng.cache.pager.free_slot_count() == 2


def test_in_step_sampling_takes_streams_and_draw_numbers_from_the_loop():
    eng = InStepEngine(None)
    sampler = ScriptedSampler(lambda s, c: 100 * s + c)
    res = Generator(eng, sampler).generate([[1], [2, 2]], max_tokens=4)
    assert [r.tokens for r in res] == [[0, 1, 2, 3], [100, 101, 102, 103]]
    assert sampler.seen == [([0, 1], [0, 0])]                      # the sampler object only after the prompts
    assert eng.sampled_in_step == [([0, 1], [1, 1]), ([0, 1], [2, 2]), ([0, 1], [3, 3])]
    assert eng.fed_in_place == 3                                   # every step read its tokens where the last one left them
    # with a token history the sampler cannot live in the step: the loop calls it after every step
    from rust_inference_b200 import SamplerConfig
    eng2 = InStepEngine(None)
    s2 = ScriptedSampler(lambda s, c: 7)
    s2.params = SamplerConfig(repetition_penalty=1.3)
    Generator(eng2, s2).generate([[1]], max_tokens=3)
    assert eng2.sampled_in_step == [] and len(s2.seen) == 3


def test_tokens_are_fed_in_place_while_the_whole_batch_goes_on():
    eng = AheadEngine()
    gen = Generator(eng, ScriptedSampler(lambda s, c: 9 if (s == 0 and c == 3) else 5), stop_ids=[9])
    res = gen.generate([[1], [2]], max_tokens=6)
    assert res[0].tokens == [5, 5, 5] and res[1].tokens == [5] * 6
    # steps of two rows were fed from the buffer the sampler wrote into (no gather, no copy); once a row
    # had been dropped, the single row that was left was gathered once, then fed in place again
    assert eng.fed_in_place >= 4
    # nothing asks for a token buffer of a size that is never stepped: the last sample of the batch
    # (and the first sample, of one row after the stop) writes to a buffer of its own
    assert set(eng.token_buffers) <= {1, 2}
    eng.cache.pager.audit()


def test_the_last_sample_of_a_batch_takes_no_token_buffer():
    eng = AheadEngine()
    Generator(eng, ScriptedSampler(lambda s, c: 5)).generate([[1], [2], [3]], max_tokens=1)
    assert eng.token_buffers == {}                               # one sample, no step after it
    eng2 = AheadEngine()
    Generator(eng2, ScriptedSampler(lambda s, c: 5)).generate([[1], [2], [3]], max_tokens=3)
    assert set(eng2.token_buffers) == {3}
