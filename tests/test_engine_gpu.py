"""The engine in process: cutting and batching invariance, slot reuse, long decoding, the first
tokens of a sequence, greedy generation through the entry point, schedules."""
import pytest
import torch

import plain_impl
from conftest import TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu


def _engine(model, dtype, **kw):
    from rust_inference_b200.engine.engine import Engine
    kw.setdefault("max_tokens", 4096)
    return Engine.from_pretrained(model.folder, dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(name, dtype, model_factory):
    """Positions 0, 1, 2: a single key, the first decoded token, a prompt of one token."""
    model = model_factory(name, std=0.08)
    eng = _engine(model, dtype)
    toks = random_tokens(6, model.cfg["vocab_size"], seed=2)
    want = model.plain_logits(toks)
    s = eng.alloc_slot()
    got = [eng.step([s], [[t]], "last")[0].cpu() for t in toks]      # token by token from position 0
    assert rel_err(torch.stack(got), want) <= TOL[dtype]
    eng.free_slot(s)
    s = eng.alloc_slot()
    first = eng.step([s], [toks[:1]], "all").cpu()                    # a prompt of one token, as prefill
    assert rel_err(first, want[:1]) <= TOL[dtype]
    rest = eng.step([s], [toks[1:]], "all").cpu()
    assert rel_err(rest, want[1:]) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_crosses_pages(dtype, model_factory):
    """300 single-token steps after a short prompt: pages are added on the way; with graphs."""
    model = model_factory("A", std=0.08)
    eng = _engine(model, dtype)
    toks = random_tokens(330, model.cfg["vocab_size"], seed=3)
    want = model.plain_logits(toks)
    s = eng.alloc_slot()
    eng.step([s], [toks[:30]], "none")
    worst = 0.0
    for i in range(30, 330):
        got = eng.step([s], [[toks[i]]], "last")[0]
        worst = max(worst, rel_err(got, want[i]))
    assert worst <= TOL[dtype]
    assert eng.cache.length(s) == 330


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_and_eager_decode_agree(dtype, model_factory):
    model = model_factory("B", std=0.08)
    a, b = _engine(model, dtype, use_graphs=True), _engine(model, dtype, use_graphs=False)
    prompts = [random_tokens(n, model.cfg["vocab_size"], seed=n) for n in (70, 5, 129)]
    sa = [a.alloc_slot() for _ in prompts]
    sb = [b.alloc_slot() for _ in prompts]
    a.step(sa, prompts, "none")
    b.step(sb, prompts, "none")
    for i in range(5):
        nxt = [[(7 * i + j) % 391] for j in range(3)]
        la, lb = a.step(sa, nxt, "last"), b.step(sb, nxt, "last")
        assert rel_err(la, lb) <= (1e-6 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_reused_slot_sees_nothing_stale(dtype, model_factory):
    """A long sequence leaves its keys in the pages; the next sequences take the same slot and
    pages and must not see them.  Large weights make attention sharp, so one stale key would
    show.  Each request must give what it gives in an engine that never held anything (equal up
    to the order of float additions), and in 32-bit also what the plain implementation gives."""
    model = model_factory("A", std=0.25)
    eng = _engine(model, dtype, max_tokens=512, n_slots=2)
    fresh = _engine(model, dtype, max_tokens=512, n_slots=2)
    vocab = model.cfg["vocab_size"]
    long_seq = random_tokens(400, vocab, seed=4)
    s = eng.alloc_slot()
    eng.step([s], [long_seq], "none")
    eng.free_slot(s)
    for n in (3, 64, 65, 130):
        toks = random_tokens(n, vocab, seed=n)
        s2 = eng.alloc_slot()
        assert s2 == s
        got = torch.cat([eng.step([s2], [toks[:-1]], "all").cpu(), eng.step([s2], [toks[-1:]], "last").cpu()])
        eng.free_slot(s2)
        f = fresh.alloc_slot()
        clean = torch.cat([fresh.step([f], [toks[:-1]], "all").cpu(), fresh.step([f], [toks[-1:]], "last").cpu()])
        fresh.free_slot(f)
        assert rel_err(got, clean) <= 1e-5, f"a reused slot changes the logits of a {n}-token request"
        if dtype == "float32":
            assert rel_err(got, model.plain_logits(toks)) <= TOL[dtype]
    eng.cache.pager.audit()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_composition_does_not_change_logits(dtype, model_factory):
    """The same request alone and inside batches of different neighbours, in different slots."""
    model = model_factory("B", std=0.08)
    eng = _engine(model, dtype)
    vocab = model.cfg["vocab_size"]
    me = random_tokens(90, vocab, seed=1)
    others = [random_tokens(n, vocab, seed=50 + n) for n in (1, 200, 64, 17)]
    s = eng.alloc_slot()
    alone = eng.step([s], [me], "all").cpu()
    eng.free_slot(s)
    slots = [eng.alloc_slot() for _ in range(5)]
    batch = eng.step(slots, others[:2] + [me] + others[2:], [[], [], list(range(90)), [], []]).cpu()
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert rel_err(batch, alone) <= tol


def test_greedy_generation_through_the_entry_point(model_factory):
    from rust_inference_b200 import Model, SamplerConfig
    model = model_factory("A", std=0.08)
    prompts = [random_tokens(n, model.cfg["vocab_size"], seed=n) for n in (5, 11, 17, 1)]
    want = [plain_impl.greedy_generate(model.weights, model.cfg, p, 8) for p in prompts]
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=1024)
    got = m.generate(prompts, 8, SamplerConfig.plain(0.0), stop_ids=())
    assert [g.tokens for g in got] == want
    assert all(g.finish_reason == "length" for g in got)
    # a stop id ends that sequence early and is not returned; the others go on
    stop = want[1][3]
    got = m.generate(prompts, 8, SamplerConfig.plain(0.0), stop_ids=(stop,))
    for g, w in zip(got, want):
        if stop in w:
            assert g.tokens == w[:w.index(stop)] and g.finish_reason == "stop"
        else:
            assert g.tokens == w and g.finish_reason == "length"
    st = m.last_stats
    assert st["generated_tokens"] == sum(len(g.tokens) for g in got) and st["prompt_tokens"] == 5 + 11 + 17 + 1
    assert st["tokens_per_second"] > 0 and st["steps"] >= 1 and st["d2h_bytes"] > 0 and st["h2d_bytes"] > 0
    mem = m.memory()
    assert mem["cache_bytes_per_position"] == 2 * 2 * 2 * 64 * 4            # 2 layers x (K, V) x 2 kv heads x 64 x float32
    assert mem["weight_bytes"] == mem["weight_bytes_per_step"]              # tied: the embedding is also the head
    # more requests than slots: batches follow one another
    m2 = Model.load(model.folder, dtype="float32", max_tokens_in_cache=256, n_slots=2)
    got = m2.generate(prompts, 8, SamplerConfig.plain(0.0), stop_ids=())
    assert [g.tokens for g in got] == want
    m2.engine.cache.pager.audit()
    # one prompt given as a plain list
    assert m.generate(prompts[0], 8, SamplerConfig.plain(0.0), stop_ids=()).tokens == want[0]
    # bf16: rows within TOL of the plain logits (relative to the row maximum) put the engine's
    # maximum within 2 TOL of the plain maximum, so that is the bound for every generated token
    mb = Model.load(model.folder, dtype="bfloat16", max_tokens_in_cache=1024)
    for p, g in zip(prompts, mb.generate(prompts, 8, SamplerConfig.plain(0.0), stop_ids=())):
        seq = list(p)
        assert len(g.tokens) == 8
        for tok in g.tokens:
            ref = model.plain_logits(seq)[-1]
            gap = float((ref.max() - ref[tok]) / ref.abs().max())
            assert gap <= 2 * TOL["bfloat16"], (tok, gap)
            seq.append(tok)


def test_greedy_generation_with_the_repetition_penalty(model_factory):
    """Penalised greedy (the reference's command line always penalises, main.rs:187-188): every step the
    logits of the last `window` ids of prompt + generated tokens are divided or multiplied by the penalty
    (sampler.rs:76-78, :109-127), then the first maximum is taken.  The generation loop runs one step
    ahead here, so the newest id of the window reaches the sampler on the device."""
    from rust_inference_b200 import Model, SamplerConfig
    model = model_factory("A", std=0.08)
    prompts = [random_tokens(n, model.cfg["vocab_size"], seed=40 + n) for n in (3, 9, 70)]
    cfg = SamplerConfig(temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.6, repetition_window=5)
    want = []
    for p in prompts:
        seq, out = list(p), []
        for _ in range(12):
            logits = plain_impl.repetition_penalty(model.plain_logits(seq)[-1], seq, 1.6, 5)
            tok = plain_impl.argmax_first(logits)
            out.append(tok)
            seq.append(tok)
        want.append(out)
    plain_greedy = [plain_impl.greedy_generate(model.weights, model.cfg, p, 12) for p in prompts]
    assert want != plain_greedy                                  # the penalty changes what is generated
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=1024)
    assert m.engine.can_feed_from_device()
    got = m.generate(prompts, 12, cfg, stop_ids=())
    assert [g.tokens for g in got] == want
    # one at a time (other batch sizes, other buffers) gives the same
    got1 = m.generate(prompts, 12, cfg, stop_ids=(), max_batch=1)
    assert [g.tokens for g in got1] == want


def test_temperature_sampling_is_reproducible_and_batch_independent(model_factory):
    from rust_inference_b200 import Model, SamplerConfig
    model = model_factory("B", std=0.08)
    prompts = [random_tokens(n, model.cfg["vocab_size"], seed=n) for n in (1, 7, 30, 64)]
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=2048)
    cfg = SamplerConfig.plain(temperature=0.7, seed=4)
    a = m.generate(prompts, 16, cfg, stop_ids=())
    b = m.generate(prompts, 16, cfg, stop_ids=())
    assert [x.tokens for x in a] == [x.tokens for x in b]
    c = m.generate(prompts, 16, SamplerConfig.plain(temperature=0.7, seed=5), stop_ids=())
    assert [x.tokens for x in a] != [x.tokens for x in c]
    # the seed lives on the device beside the draw counters: another seed took no other capture
    assert m.engine.decode_graph(4, cfg) is m.engine.decode_graph(4, SamplerConfig.plain(temperature=0.7, seed=5))
    assert m.engine.decode_graph(4, cfg).graph is not None
    # a seed beyond 32 bits, checked against the host's restatement of the draw
    from conftest import oracle_generate
    big = SamplerConfig.plain(temperature=0.7, seed=0x1234_5678_9ABC_DEF1)
    e = m.generate(prompts[:2], 6, big, stop_ids=())
    for i, p in enumerate(prompts[:2]):
        assert e[i].tokens == oracle_generate(model, p, 6, temperature=0.7, seed=big.seed, stream=i)
    # request 2 draws the same numbers when the batch is cut differently (one at a time)
    d = m.generate(prompts, 16, cfg, stop_ids=(), max_batch=1)
    assert [x.tokens for x in d] == [x.tokens for x in a]


def test_device_resident_decode_matches_the_loop(model_factory):
    from rust_inference_b200 import Model, SamplerConfig
    model = model_factory("A", std=0.08)
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=1024)
    prompts = [random_tokens(n, model.cfg["vocab_size"], seed=n) for n in (9, 70)]
    want = m.generate(prompts, 10, SamplerConfig.plain(0.0), stop_ids=())
    eng = m.engine
    slots = [eng.alloc_slot() for _ in prompts]
    eng.step(slots, [p[:-1] for p in prompts], "none")
    toks = eng.decode_steps(slots, [p[-1] for p in prompts], 10).cpu()
    assert toks.t().tolist() == [w.tokens for w in want]


def test_step_refuses_bad_input(model_factory):
    from rust_inference_b200.cache.pager import CacheError, CacheFull
    model = model_factory("A", std=0.08)
    eng = _engine(model, "float32", max_tokens=128, n_slots=2)
    s = eng.alloc_slot()
    with pytest.raises(ValueError, match="token id"):
        eng.step([s], [[1, 264]], "last")
    with pytest.raises(ValueError, match="twice"):
        eng.step([s, s], [[1], [2]], "last")
    with pytest.raises(ValueError, match="no tokens"):
        eng.step([s], [[]], "last")
    with pytest.raises(CacheFull):
        eng.step([s], [[1] * 200], "last")
    with pytest.raises(CacheError):
        eng.step([1], [[1]], "last")                       # slot 1 was never handed out
    assert eng.cache.length(s) == 0                        # nothing was committed
    out = eng.step([s], [[1, 2, 3]], [[1]])
    assert out.shape == (1, 264)
    assert eng.step([s], [[4]], "none") is None
    with pytest.raises(RuntimeError, match="CUDA"):
        from rust_inference_b200.engine.engine import Engine
        Engine.from_pretrained(model.folder, dtype="float32", device="cpu", max_tokens=64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_order_of_layers_is_data(dtype, model_factory):
    """A schedule that runs a layer twice, and one in which a layer reads another layer's keys
    and values, against the plain implementation given the same list."""
    import dataclasses
    from rust_inference_b200 import load_config
    from rust_inference_b200.config.registry import get_architecture
    from rust_inference_b200.engine.engine import Engine
    from rust_inference_b200.engine.model import DecoderModel
    from rust_inference_b200.parts.spec import ScheduleEntry
    from rust_inference_b200.weights.loader import read_model_tensors
    model = model_factory("A", std=0.08)
    cfg = load_config(model.folder)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    toks = random_tokens(80, cfg.vocab_size, seed=8)
    cases = {
        "twice": ([ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2)], [(0, None), (1, None), (0, None)]),
        "shared": ([ScheduleEntry(0, 0), ScheduleEntry(1, 0)], [(0, None), (1, 0)]),
    }
    for label, (schedule, plain_schedule) in cases.items():
        s2 = dataclasses.replace(spec, schedule=tuple(schedule))
        dm = DecoderModel(s2, dtype=torch.float32 if dtype == "float32" else torch.bfloat16, device="cuda")
        dm.load(read_model_tensors(model.folder, dm.declared_tensors()))
        eng = Engine(dm, max_tokens=512)
        want = model.plain_logits(toks, schedule=plain_schedule)
        slot = eng.alloc_slot()
        head = eng.step([slot], [toks[:50]], "all").cpu()
        tail = torch.cat([eng.step([slot], [[t]], "last").cpu() for t in toks[50:]])
        assert rel_err(torch.cat([head, tail]), want) <= TOL[dtype], label


def test_a_failed_decode_step_leaves_no_dirty_accumulator(model_factory, monkeypatch):
    """A bf16 decode step of a model this wide adds the pieces of its K-split q/k/v projection onto a
    float32 accumulator that the rotary kernel consumes and zeroes again.  If a step fails between the two, the
    accumulator must not keep the leftovers: the failure is injected on the host (the rotary kernel's
    Python face raises before it launches), in each phase of a batch size's life: on the engine's
    shared scratch, on the size's own scratch, during the capture, and in a replayed graph's neighbour
    (an eager prefill step)."""
    from rust_inference_b200.kernels import ops, tcgen05
    model = model_factory("E", std=0.05)
    eng = _engine(model, "bfloat16")
    assert tcgen05.plan(5, 8 * 64 + 2 * 2 * 64, 512, ops.EPI_RESIDUAL)[1] > 1     # the projection is split over K
    n = 5
    seqs = [random_tokens(60, model.cfg["vocab_size"], seed=8 + i) for i in range(n)]
    want = [model.plain_logits(t) for t in seqs]
    slots = [eng.alloc_slot() for _ in range(n)]
    eng.step(slots, [t[:40 - i] for i, t in enumerate(seqs)], "none")
    at = [40 - i for i in range(n)]
    real = ops.rope_cache_write_acc
    state = {"fail": False, "calls": 0}

    def flaky(*a, **k):
        state["calls"] += 1
        if state["fail"]:
            raise RuntimeError("injected")
        return real(*a, **k)

    monkeypatch.setattr(ops, "rope_cache_write_acc", flaky)
    step = lambda: eng.step(slots, [[seqs[i][at[i]]] for i in range(n)], "last")
    # decode steps of this batch size, in order: the 1st and 2nd run on the engine's shared scratch, the
    # 3rd on the size's own, the 4th is captured; after an abandoned capture the next step captures again
    for nth, outcome in enumerate(["fail", "ok", "fail", "fail", "ok", "ok", "ok"], start=1):
        if outcome == "fail":
            state["fail"] = True
            with pytest.raises(RuntimeError, match="injected"):
                step()
            state["fail"] = False
            assert eng.cache.lengths(slots) == at              # the failed step did not count
            assert eng.decode_graph(n).graph is None
            continue
        got = step().cpu()
        for i in range(n):
            assert rel_err(got[i], want[i][at[i]]) <= TOL["bfloat16"], (nth, i)
            at[i] += 1
    assert eng.decode_graph(n).graph is not None               # the size did get its graph in the end
    assert state["calls"] > 0                                  # the path under test did run
    # an eager step of several tokens that fails, then the same step again
    s, pos, toks = slots[0], at[0], seqs[0]
    state["fail"] = True
    with pytest.raises(RuntimeError, match="injected"):
        eng.step([s], [toks[pos:pos + 5]], "all")
    state["fail"] = False
    got = eng.step([s], [toks[pos:pos + 5]], "all")
    assert rel_err(got, want[0][pos:pos + 5]) <= TOL["bfloat16"]
    eng.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_random_model_saved_and_loaded_again(dtype, tmp_path):
    """`Model.random` makes its weights on the device; `state_dict()` hands them to the plain
    implementation without a folder, and `save_safetensors` writes a folder that loads to the same logits."""
    from conftest import TINY
    from rust_inference_b200 import Model, config_from_dict
    cfg = config_from_dict(TINY["B"])
    m = Model.random(cfg, seed=12, std=0.08, norm_std=0.2, dtype=dtype, max_tokens_in_cache=512)
    toks = random_tokens(40, cfg.vocab_size, seed=1)
    weights = {n: t.float().cpu() for n, t in m.state_dict().items()}
    want = plain_impl.forward(weights, cfg.to_dict(), toks)
    got = m.logits(toks)
    assert rel_err(got, want) <= TOL[dtype]
    # the device-made weights are a function of (seed, tensor name, element) that the host can restate
    import zlib
    from rust_inference_b200.sampling import rng
    name = "model.layers.1.mlp.down_proj.weight"
    key = (12 * 1_000_003 + zlib.crc32(name.encode())) % (2 ** 63 - 1)
    got_w = m.state_dict()[name].float().flatten().cpu()
    for i in (0, 5, got_w.numel() - 1):
        assert abs(float(got_w[i]) - 0.08 * rng.normal(key, i)) <= (1e-6 if dtype == "float32" else 1e-3)
    folder = m.save_safetensors(str(tmp_path / "saved"))
    again = Model.load(folder, dtype=dtype, max_tokens_in_cache=512).logits(toks)
    assert rel_err(again, got) <= (1e-6 if dtype == "float32" else 2e-2)


def test_bfloat16_generation_with_stop_ids(model_factory):
    """bfloat16, greedy, stop ids, batches that shrink and follow one another: a run with stop ids is the
    free run cut before each sequence's first stop id (model.rs:383-387), and every token of the free run
    is within the bfloat16 bound of the plain implementation's maximum."""
    from rust_inference_b200 import Model, SamplerConfig
    model = model_factory("B", std=0.08)
    vocab = model.cfg["vocab_size"]
    prompts = [random_tokens(n, vocab, seed=300 + n) for n in (3, 41, 8, 1, 66, 17, 5)]
    greedy = SamplerConfig.plain(0.0)
    m = Model.load(model.folder, dtype="bfloat16", max_tokens_in_cache=1024, n_slots=4)
    free = [r.tokens for r in m.generate(prompts, 14, greedy, stop_ids=())]
    for p, toks in zip(prompts[:3], free[:3]):
        seq = list(p)
        for tok in toks:
            ref = model.plain_logits(seq)[-1]
            assert float((ref.max() - ref[tok]) / ref.abs().max()) <= 2 * TOL["bfloat16"]
            seq.append(tok)
    stops = (free[0][4], free[1][0], free[4][9], free[6][13])          # an early one, a first token, a late one, a last one
    got = m.generate(prompts, 14, greedy, stop_ids=stops)
    n_stopped = 0
    for g, f in zip(got, free):
        cut = next((i for i, t in enumerate(f) if t in stops), None)
        if cut is None:
            assert g.tokens == f and g.finish_reason == "length"
        else:
            assert g.tokens == f[:cut] and g.finish_reason == "stop"
            n_stopped += 1
    assert n_stopped >= 4
    m.engine.cache.pager.audit()
    assert m.engine.cache.pager.free_slot_count() == 4
    m.engine.check_device_status()
