"""Each part alone against the plain function of the same part, and a toy mixer with state of
its own that is registered, built and stepped without touching the library's files."""
import math

import pytest
import torch

import plain_impl
from conftest import random_tokens, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ctx(starts, tokens, cache, dtype):
    """A step context for parts tested outside an engine."""
    from rust_inference_b200.engine.context import StepContext, Workspace, pack_step
    wants = [list(range(len(t))) for t in tokens]
    meta, layout, sc = pack_step(starts, tokens, wants)
    o, c = layout["seq_slot"]
    slots = [cache.alloc_slot() for _ in tokens]
    meta[o:o + c] = slots
    cache.reserve([(s, st + len(t)) for s, st, t in zip(slots, starts, tokens)])
    dev = torch.from_numpy(meta).to(DEV)
    v = lambda name: dev[layout[name][0]:layout[name][0] + layout[name][1]]
    return StepContext(
        n_tokens=sc["n_tokens"], n_seqs=sc["n_seqs"], token_ids=v("token_ids"), token_pos=v("token_pos"),
        token_seq=v("token_seq"), seq_slot=v("seq_slot"), seq_start=v("seq_start"), seq_len=v("seq_len"),
        cu_seqlens=v("cu_seqlens"), logit_rows=v("logit_rows"), n_logit_rows=sc["n_logit_rows"],
        max_new=sc["max_new"], max_len=sc["max_len"], all_single=sc["all_single"], page_table=cache.page_table,
        page_size=cache.page_size, dtype=dtype, device=torch.device(DEV), workspace=Workspace(DEV))


def _place(part, tensors, dtype):
    placed = {}
    for name, ts in part.tensor_specs().items():
        t = tensors[name]
        placed[name] = t.to(DEV, dtype if ts.role == "matrix" else torch.float32).contiguous()
    part.set_tensors(placed)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from rust_inference_b200.parts.registry import lookup
    part = lookup("norm", "rmsnorm")(eps=3e-4, hidden_size=200, dtype=dtype, device=DEV)
    assert part.tensor_specs()["weight"].shape == (200,) and part.tensor_specs()["weight"].init == "ones"
    w = torch.randn(200)
    _place(part, {"weight": w}, dtype)
    x = torch.randn(11, 200, device=DEV)
    out = torch.empty(11, 200, device=DEV, dtype=dtype)
    part.forward(x, out)
    want = plain_impl.rmsnorm(x.cpu(), w, 3e-4)
    assert rel_err(out, want) <= (1e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from rust_inference_b200.parts.registry import lookup
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    h, inter, n = 96, 200, 37
    part = lookup("feed_forward", "swiglu")(intermediate_size=inter, hidden_size=h, dtype=dtype, device=DEV)
    p = {"gate_proj.weight": torch.randn(inter, h) * 0.2, "up_proj.weight": torch.randn(inter, h) * 0.2,
         "down_proj.weight": torch.randn(h, inter) * 0.2}
    p = {k: v.to(dtype).float() for k, v in p.items()}
    _place(part, p, dtype)
    cache = SequenceCache([], max_tokens=64, max_seq_len=64, dtype=dtype, device=DEV)
    ctx = _ctx([0], [list(range(n))], cache, dtype)
    x = (torch.randn(n, h) * 0.5).to(dtype)
    residual = torch.randn(n, h, device=DEV)
    before = residual.clone().cpu()
    part.forward(x.to(DEV), residual, ctx)
    want = before + plain_impl.swiglu(x.float(), p, "")
    assert rel_err(residual, want) <= (2e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("style, bias, nh, nkv, hd, h", [
    ("half", False, 4, 2, 64, 80), ("interleaved", True, 6, 1, 32, 80), ("half", True, 3, 3, 128, 80),
    # a width at which the single-token projections are split over K into float32 accumulators
    ("half", True, 4, 2, 64, 1536), ("interleaved", False, 2, 1, 128, 1024)])
def test_attention_part_with_cache(dtype, style, bias, nh, nkv, hd, h):
    """The mixer alone: a prompt in one step and then token by token must equal the plain
    attention over the whole sequence."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.kernels import linear
    from rust_inference_b200.parts.registry import lookup
    from rust_inference_b200.parts.spec import PartSpec
    n, cut = 150, 100
    part = lookup("mixer", "gqa_attention")(
        n_heads=nh, n_kv_heads=nkv, head_dim=hd, qkv_bias=bias,
        position=PartSpec("rope", {"head_dim": hd, "base": 50000.0, "style": style}),
        hidden_size=h, dtype=dtype, device=DEV)
    specs = part.tensor_specs()
    assert ("q_proj.bias" in specs) == bias and specs["k_proj.weight"].shape == (nkv * hd, h)
    p = {name: (torch.randn(ts.shape) * ((2.0 / h ** 0.5) if ts.role == "matrix" else 0.1)).to(dtype).float()
         for name, ts in specs.items()}
    _place(part, p, dtype)
    part.prepare(256)
    one = torch.zeros(1, h, device=DEV, dtype=dtype)
    assert linear.wants_split(one, part.w_qkv) == (dtype == torch.bfloat16 and h >= 1024)
    cache = SequenceCache([part.cache_request()], max_tokens=512, max_seq_len=256, dtype=dtype, device=DEV)
    x = (torch.randn(n, h) * 0.5).to(dtype)
    cos, sin = plain_impl.rope_table(hd, 50000.0, n)
    want, _ = plain_impl.attention(x.float(), p, "", n_heads=nh, n_kv_heads=nkv, head_dim=hd, cos=cos, sin=sin,
                                   rope_style=style)
    ctx = _ctx([0], [list(range(cut))], cache, dtype)
    slot = int(ctx.seq_slot[0])
    got = torch.zeros(n, h, device=DEV)
    part.forward(x[:cut].to(DEV), got[:cut], ctx, cache.layer(0), True)
    cache.commit(slot, cut)
    from rust_inference_b200.engine.context import pack_step
    for i in range(cut, n):
        meta, layout, sc = pack_step([i], [[0]], [[0]])
        meta[layout["seq_slot"][0]] = slot
        cache.reserve([(slot, i + 1)])
        dev = torch.from_numpy(meta).to(DEV)
        for name in ("token_pos", "token_seq", "seq_slot", "seq_start", "seq_len", "cu_seqlens"):
            o, c = layout[name]
            setattr(ctx, name, dev[o:o + c])
        ctx.n_tokens, ctx.n_seqs, ctx.max_new, ctx.max_len, ctx.all_single = 1, 1, 1, i + 1, True
        part.forward(x[i:i + 1].to(DEV), got[i:i + 1], ctx, cache.layer(0), True)
        cache.commit(slot, i + 1)
    assert rel_err(got, want) <= (1e-5 if dtype == torch.float32 else 2e-2)


def test_rope_part_needs_prepared_tables():
    from rust_inference_b200.parts.registry import lookup
    part = lookup("position", "rope")(head_dim=16, base=1e4, style="half", hidden_size=32, dtype=torch.float32,
                                      device=DEV)
    part.prepare(10)
    assert part.cos.shape == (10, 8) and part.cos.dtype == torch.float32
    with pytest.raises(ValueError):
        lookup("position", "rope")(head_dim=15, base=1e4, hidden_size=32, dtype=torch.float32, device=DEV)
    with pytest.raises(KeyError, match="no mixer registered"):
        lookup("mixer", "nonexistent")


# ------------------------------------------------------------------------------------------
# A toy mixer with state of its own, defined here, registered from outside the package.
# It keeps a running mean of its inputs per sequence: out_t = W * mean(x_0..x_t).  Its state
# (the running sum and the count) lives in the cache's fixed-size per-sequence state area.
# ------------------------------------------------------------------------------------------
def _register_toy():
    from rust_inference_b200.cache.sequence_cache import StateRequest
    from rust_inference_b200.parts.base import Mixer
    from rust_inference_b200.parts.registry import register
    from rust_inference_b200.parts.spec import TensorSpec

    @register("mixer", "toy_running_mean", replace=True)
    class RunningMean(Mixer):
        graph_safe = False        # loops over the sequences on the host

        def __init__(self, *, gain: float, hidden_size, dtype, device):
            super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
            self.gain = gain
            self.w = None

        def tensor_specs(self):
            return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size))}

        def set_tensors(self, tensors):
            self.w = tensors["mix.weight"]

        def cache_request(self):
            return StateRequest((self.hidden_size + 1,), torch.float32)      # running sum, count

        def forward(self, x, residual, ctx, cache_layer, writes_cache):
            state = cache_layer.state                                         # [slots, hidden + 1]
            slots, cu = ctx.host_slots, [0]
            for n in ctx.host_counts:
                cu.append(cu[-1] + n)
            for b, slot in enumerate(slots):
                xs = x[cu[b]:cu[b + 1]].float()
                sums = state[slot, :-1] + torch.cumsum(xs, dim=0)
                counts = state[slot, -1] + torch.arange(1, xs.shape[0] + 1, device=x.device)
                residual[cu[b]:cu[b + 1]] += self.gain * ((sums / counts[:, None]) @ self.w.float().t())
                if writes_cache:
                    state[slot, :-1] = sums[-1]
                    state[slot, -1] = counts[-1]
    return RunningMean


def _toy_architecture():
    from rust_inference_b200.config.registry import register_architecture
    from rust_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    def parse(d):
        return d

    def build(d):
        rope = PartSpec("rope", {"head_dim": 64, "base": 1e4, "style": "half"})
        attn = PartSpec("gqa_attention", {"n_heads": 2, "n_kv_heads": 1, "head_dim": 64, "qkv_bias": False,
                                          "position": rope}, prefix="attn.")
        toy = PartSpec("toy_running_mean", {"gain": d["gain"]}, prefix="toy.")
        ff = PartSpec("swiglu", {"intermediate_size": d["inter"]}, prefix="ff.")
        norm = lambda p: PartSpec("rmsnorm", {"eps": 1e-5}, prefix=p)
        layers = tuple(LayerSpec(prefix=f"l{i}.", mixer=m, feed_forward=ff, mixer_norm=norm("n1."),
                                 feed_forward_norm=norm("n2.")) for i, m in enumerate([toy, attn, toy]))
        return ModelSpec(hidden_size=d["hidden"], vocab_size=d["vocab"], max_positions=512, layers=layers,
                         schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 2)),
                         final_norm=PartSpec("rmsnorm", {"eps": 1e-5}, prefix="final."),
                         embedding_name="embed.weight", head_name="head.weight")

    register_architecture("ToyStateLM", parse, build, replace=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_registers_builds_and_steps(dtype, tmp_path):
    """Different mixers in different layers of one model; the toy's state follows the slot:
    cutting a sequence into steps, batching it with others and reusing its slot change nothing."""
    import json
    import os
    from rust_inference_b200.cache.sequence_cache import KVRequest, StateRequest
    from rust_inference_b200.config.registry import unregister_architecture
    from rust_inference_b200.engine.engine import Engine
    from rust_inference_b200.engine.model import declared_tensors
    from rust_inference_b200.parts.registry import unregister
    from rust_inference_b200.weights.loader import random_tensors
    from rust_inference_b200.weights.safetensors_io import write_safetensors
    from rust_inference_b200.config.registry import get_architecture

    _register_toy()
    _toy_architecture()
    try:
        cfg = {"architectures": ["ToyStateLM"], "hidden": 64, "inter": 96, "vocab": 50, "gain": 0.5}
        folder = str(tmp_path / "toy")
        os.makedirs(folder)
        json.dump(cfg, open(os.path.join(folder, "config.json"), "w"))
        spec = get_architecture("ToyStateLM").build_spec(cfg)
        names = declared_tensors(spec)
        assert "l0.toy.mix.weight" in names and "l1.attn.q_proj.weight" in names and "l2.toy.mix.weight" in names
        write_safetensors(os.path.join(folder, "model.safetensors"), dict(random_tensors(names, 0, std=0.1, norm_std=0.2)))
        eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=1024, n_slots=3)
        reqs = eng.model.cache_requests()
        assert isinstance(reqs[0], StateRequest) and isinstance(reqs[1], KVRequest) and reqs[0] == reqs[2]
        assert len(eng.cache.groups) == 2                     # state layers share one group, kv has its own

        toks = random_tokens(90, 50, seed=1)
        other = random_tokens(40, 50, seed=2)
        s = eng.alloc_slot()
        whole = eng.step([s], [toks], "all").cpu()
        eng.free_slot(s)
        # the same slot again (its state must start from zero), now cut into unequal steps inside a batch
        s, o = eng.alloc_slot(), eng.alloc_slot()
        parts = [eng.step([o, s], [other[:7], toks[:33]], [[], list(range(33))]).cpu()]
        parts.append(eng.step([s, o], [toks[33:60], other[7:]], [list(range(27)), []]).cpu())
        parts += [eng.step([s], [[t]], "last").cpu() for t in toks[60:]]
        tol = 1e-5 if dtype == "float32" else 3e-2
        assert rel_err(torch.cat(parts), whole) <= tol
        # and the state does something: without the toy layers' state the logits differ
        assert eng.cache.layer(0).state[s].abs().sum() > 0
    finally:
        unregister("mixer", "toy_running_mean")
        unregister_architecture("ToyStateLM")
