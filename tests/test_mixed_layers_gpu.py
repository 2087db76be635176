"""One model whose layers differ, assembled from parts by an architecture that is defined here and
registered from outside the package:

  layer 0  attention over all keys, 4 heads over 2 kv heads of 64, biases, half-split rotary
           (base 1e4); SwiGLU of width 176
  layer 1  attention over a window of 24 keys, 2 heads over 1 kv head of 128, no biases,
           interleaved rotary (base 1e6), another eps; SwiGLU of width 96
  layer 2  attention over all keys, 4 heads over 4 kv heads of 32; a toy feed-forward with routing
           (top-1 of 3 small experts), defined here
  layer 3  a toy mixer without position encoding that adds a learned per-position vector (another
           way for positions to enter), defined here; SwiGLU of width 64

The engine is compared with the plain implementation's parts put together the same way: whole,
with the last tokens one by one, and in a batch of unequal lengths with a slot used again."""
import json
import os

import pytest
import torch

import plain_impl
from conftest import oracle_weights, random_tokens, rel_err
from conftest import rel_err as _rel_err

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, MAX_POS = 128, 211, 256
LAYERS = [
    dict(nh=4, nkv=2, hd=64, bias=True, style="half", base=1e4, window=None, eps=1e-5, inter=176),
    dict(nh=2, nkv=1, hd=128, bias=False, style="interleaved", base=1e6, window=24, eps=1e-6, inter=96),
    dict(nh=4, nkv=4, hd=32, bias=False, style="half", base=5e5, window=None, eps=1e-5, experts=3, inter=48),
    dict(eps=1e-5, inter=64),
]


def _register_parts():
    from rust_inference_b200.kernels import linear
    from rust_inference_b200.parts.base import FeedForward, Mixer
    from rust_inference_b200.parts.registry import register
    from rust_inference_b200.parts.spec import TensorSpec

    @register("feed_forward", "toy_routed", replace=True)
    class ToyRouted(FeedForward):
        """Router logits in float32, the best expert per token (the first on ties), its SwiGLU
        output weighted by the softmax probability of the choice."""
        graph_safe = False        # picks each expert's tokens on the host

        def __init__(self, *, n_experts: int, intermediate_size: int, hidden_size, dtype, device):
            super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
            self.n_experts, self.inter = n_experts, intermediate_size
            self.router = None
            self.experts = []

        def tensor_specs(self):
            specs = {"router.weight": TensorSpec((self.n_experts, self.hidden_size), role="vector")}
            for e in range(self.n_experts):
                specs[f"experts.{e}.gate_proj.weight"] = TensorSpec((self.inter, self.hidden_size))
                specs[f"experts.{e}.up_proj.weight"] = TensorSpec((self.inter, self.hidden_size))
                specs[f"experts.{e}.down_proj.weight"] = TensorSpec((self.hidden_size, self.inter))
            return specs

        def set_tensors(self, tensors):
            self.router = tensors["router.weight"]                       # float32 (role "vector")
            self.experts = [tuple(linear.Weight(tensors[f"experts.{e}.{n}_proj.weight"]) for n in ("gate", "up", "down"))
                            for e in range(self.n_experts)]

        def forward(self, x, residual, ctx):
            probs = torch.softmax(x.float() @ self.router.t(), dim=-1)
            best = probs.argmax(dim=-1)
            for e, (gate, up, down) in enumerate(self.experts):
                rows = (best == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                xe = x[rows].contiguous()
                act = torch.empty(xe.shape[0], self.inter, dtype=self.dtype, device=x.device)
                linear.gated(xe, gate, up, act, ctx)
                out = torch.zeros(xe.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
                linear.into_residual(act, down, out, ctx)
                residual[rows] += probs[rows, e][:, None] * out

    @register("mixer", "toy_position_add", replace=True)
    class PositionAdd(Mixer):
        """residual += table[position]: learned absolute positions, no cache of its own."""

        def __init__(self, *, max_positions: int, hidden_size, dtype, device):
            super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
            self.max_positions = max_positions
            self.table = None

        def tensor_specs(self):
            return {"positions.weight": TensorSpec((self.max_positions, self.hidden_size), role="vector")}

        def set_tensors(self, tensors):
            self.table = tensors["positions.weight"]

        def forward(self, x, residual, ctx, cache_layer, writes_cache):
            residual += self.table[ctx.token_pos.long()]


def _register_architecture():
    from rust_inference_b200.config.registry import register_architecture
    from rust_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, default_schedule

    def build(d):
        layers = []
        for i, L in enumerate(d["layers"]):
            norm = lambda p: PartSpec("rmsnorm", {"eps": L["eps"]}, prefix=p)
            if "nh" in L:
                rope = PartSpec("rope", {"head_dim": L["hd"], "base": L["base"], "style": L["style"]})
                mixer = PartSpec("gqa_attention", {"n_heads": L["nh"], "n_kv_heads": L["nkv"], "head_dim": L["hd"],
                                                   "qkv_bias": L["bias"], "position": rope, "window": L["window"]},
                                 prefix="self_attn.")
            else:
                mixer = PartSpec("toy_position_add", {"max_positions": d["max_positions"]}, prefix="pos.")
            if "experts" in L:
                ff = PartSpec("toy_routed", {"n_experts": L["experts"], "intermediate_size": L["inter"]}, prefix="moe.")
            else:
                ff = PartSpec("swiglu", {"intermediate_size": L["inter"]}, prefix="mlp.")
            layers.append(LayerSpec(prefix=f"model.layers.{i}.", mixer=mixer, feed_forward=ff,
                                    mixer_norm=norm("input_layernorm."), feed_forward_norm=norm("post_attention_layernorm.")))
        return ModelSpec(hidden_size=d["hidden"], vocab_size=d["vocab"], max_positions=d["max_positions"],
                         layers=tuple(layers), schedule=default_schedule(len(layers)),
                         final_norm=PartSpec("rmsnorm", {"eps": 1e-5}, prefix="model.norm."),
                         embedding_name="model.embed_tokens.weight", head_name="lm_head.weight")

    register_architecture("ToyMixedLM", lambda d: d, build, replace=True)


def _plain_logits(w: dict, tokens, dtype=torch.float32, margins: list | None = None):
    """The same stack from the plain implementation's parts, one whole sequence.  `margins` receives,
    per position, how far the routed layer's best expert leads the second best (difference of their
    router logits over the largest |logit|): a choice that hangs on less than bfloat16's rounding of
    the router's input is no test of a bfloat16 run."""
    p = {k: v.to(dtype) for k, v in w.items()}
    n = len(tokens)
    h = plain_impl.embedding(p["model.embed_tokens.weight"], tokens)
    for i, L in enumerate(LAYERS):
        pre = f"model.layers.{i}."
        xn = plain_impl.rmsnorm(h, p[pre + "input_layernorm.weight"], L["eps"])
        if "nh" in L:
            cos, sin = plain_impl.rope_table(L["hd"], L["base"], n, dtype=dtype)
            a, _ = plain_impl.attention(xn, p, pre + "self_attn.", n_heads=L["nh"], n_kv_heads=L["nkv"],
                                        head_dim=L["hd"], cos=cos.to(h.device), sin=sin.to(h.device),
                                        rope_style=L["style"], window=L["window"])
        else:
            a = p[pre + "pos.positions.weight"][:n]
        h = h + a
        xn = plain_impl.rmsnorm(h, p[pre + "post_attention_layernorm.weight"], L["eps"])
        if "experts" in L:
            router_logits = plain_impl.linear(xn.float(), w[pre + "moe.router.weight"].float().to(h.device))
            probs = plain_impl.softmax_rows(router_logits)
            if margins is not None:
                top = router_logits.topk(2, dim=-1).values
                margins.extend(((top[:, 0] - top[:, 1]) / router_logits.abs().amax(dim=-1)).tolist())
            out = torch.zeros_like(h)
            for t in range(n):
                e = plain_impl.argmax_first(probs[t])
                out[t] = probs[t, e].to(dtype) * plain_impl.swiglu(xn[t:t + 1], p, pre + f"moe.experts.{e}.")[0]
            h = h + out
        else:
            h = h + plain_impl.swiglu(xn, p, pre + "mlp.")
    h = plain_impl.rmsnorm(h, p["model.norm.weight"], 1e-5)
    return plain_impl.linear(h, p["lm_head.weight"])


@pytest.fixture(scope="module")
def mixed_model(tmp_path_factory):
    from rust_inference_b200.config.registry import get_architecture, unregister_architecture
    from rust_inference_b200.engine.model import declared_tensors
    from rust_inference_b200.parts.registry import unregister
    from rust_inference_b200.weights.loader import random_tensors
    from rust_inference_b200.weights.safetensors_io import write_safetensors
    _register_parts()
    _register_architecture()
    folder = str(tmp_path_factory.mktemp("mixed") / "model")
    os.makedirs(folder)
    cfg = {"architectures": ["ToyMixedLM"], "hidden": HIDDEN, "vocab": VOCAB, "max_positions": MAX_POS, "layers": LAYERS}
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = declared_tensors(get_architecture("ToyMixedLM").build_spec(cfg))
    tensors = dict(random_tensors(names, 3, std=0.08, norm_std=0.2))
    # a decisive router: the best expert of a token must not hang on bfloat16's rounding of its input
    tensors["model.layers.2.moe.router.weight"] *= 6.0
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    weights = oracle_weights(folder)
    yield folder, weights
    unregister("feed_forward", "toy_routed")
    unregister("mixer", "toy_position_add")
    unregister_architecture("ToyMixedLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_that_differ_in_one_model(dtype, mixed_model):
    from rust_inference_b200.cache.sequence_cache import KVRequest
    from rust_inference_b200.engine.engine import Engine
    folder, weights = mixed_model
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=1024, n_slots=4)
    reqs = eng.model.cache_requests()
    assert reqs[:3] == [KVRequest(2, 64, None), KVRequest(1, 128, 24), KVRequest(4, 32, None)] and reqs[3] is None
    assert len(eng.cache.groups) == 3                       # every attention layer has needs of its own
    assert not eng.model.graph_safe()                       # the routed feed-forward needs the host

    tol = 1e-4 if dtype == "float32" else 4e-2
    toks = random_tokens(100, VOCAB, seed=11)

    def plain(tokens):
        """(logits, rows to compare): in bfloat16 only the positions whose expert is chosen by a clear
        margin; no layer after the routed one mixes positions, so the others do not disturb them."""
        margins = []
        logits = _plain_logits(weights, tokens, margins=margins)
        decided = torch.tensor(margins) > 0.05 if dtype == "bfloat16" else torch.ones(len(tokens), dtype=torch.bool)
        assert decided.float().mean() > 0.7
        return logits, decided

    def rel_err(got, pair, upto=None, start=0):
        logits, decided = pair
        rows = decided[start:upto]
        return _rel_err(got[rows], logits[start:upto][rows])

    want = plain(toks)
    # whole, then the last 32 one by one
    s = eng.alloc_slot()
    whole = eng.step([s], [toks], "all").cpu()
    eng.free_slot(s)
    assert rel_err(whole, want) <= tol
    s = eng.alloc_slot()
    head = eng.step([s], [toks[:68]], "all").cpu()
    tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in toks[68:]])
    eng.free_slot(s)
    assert rel_err(torch.cat([head, tail]), want) <= tol
    # the window does something: with all keys visible in layer 1 the late logits differ
    saved = LAYERS[1]["window"]
    LAYERS[1]["window"] = None
    try:
        unwindowed = _plain_logits(weights, toks)
    finally:
        LAYERS[1]["window"] = saved
    assert _rel_err(unwindowed[60:], want[0][60:]) > 10 * tol

    # a batch of unequal lengths; the shortest ends first and its slot is used again
    others = [random_tokens(n, VOCAB, seed=20 + n) for n in (9, 37)]
    slots = [eng.alloc_slot() for _ in range(3)]
    seqs = [toks[:50], others[0], others[1]]
    got = eng.step(slots, [q[:-4] for q in seqs], "all").cpu()
    rows, at = {}, 0
    for i, q in enumerate(seqs):
        rows[i] = [got[at:at + len(q) - 4]]
        at += len(q) - 4
    for step in range(4):
        live = [i for i in range(3) if not (i == 1 and step >= 2)]            # sequence 1 ends two steps early
        out = eng.step([slots[i] for i in live], [[seqs[i][len(seqs[i]) - 4 + step]] for i in live], "last").cpu()
        for j, i in enumerate(live):
            rows[i].append(out[j:j + 1])
        if step == 1:
            eng.free_slot(slots[1])
            again = eng.alloc_slot()
            assert again == slots[1]
            fresh = eng.step([again], [toks[:30]], "all").cpu()
            assert rel_err(fresh, want, upto=30) <= tol
            eng.free_slot(again)
    assert rel_err(torch.cat(rows[0]), want, upto=50) <= tol
    assert rel_err(torch.cat(rows[2]), plain(others[1])) <= tol
    assert rel_err(torch.cat(rows[1]), plain(others[0]), upto=len(others[0]) - 2) <= tol
    eng.check_device_status()


# ------------------------------------------------------------------------------------------
# Another norm and another arrangement, defined here: a LayerNorm with a bias (mean subtracted), and
# a block that feeds the same normalised input to the mixer and to the feed-forward and adds both
# to the stream (h = x + mix(norm(x)) + ff(norm(x))).  Registered from outside the package, built
# from a spec and stepped like any other model.
# ------------------------------------------------------------------------------------------
def _register_parallel():
    from rust_inference_b200.config.registry import register_architecture
    from rust_inference_b200.parts.base import Arrangement, Norm
    from rust_inference_b200.parts.registry import register
    from rust_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, TensorSpec, default_schedule

    @register("norm", "toy_layernorm", replace=True)
    class ToyLayerNorm(Norm):
        graph_safe = True

        def __init__(self, *, eps: float, hidden_size, dtype, device):
            super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
            self.eps = eps
            self.weight = self.bias = None

        def tensor_specs(self):
            return {"weight": TensorSpec((self.hidden_size,), role="vector", init="ones"),
                    "bias": TensorSpec((self.hidden_size,), role="vector")}

        def set_tensors(self, tensors):
            self.weight, self.bias = tensors["weight"], tensors["bias"]

        def forward(self, x, out, rows=None):
            src = x if rows is None else x[rows.long()]
            mean = src.mean(dim=-1, keepdim=True)
            var = ((src - mean) ** 2).mean(dim=-1, keepdim=True)
            out.copy_(((src - mean) / torch.sqrt(var + self.eps) * self.weight + self.bias).to(out.dtype))
            return out

    @register("arrangement", "toy_parallel", replace=True)
    class Parallel(Arrangement):
        def forward(self, residual, ctx, cache_layer, writes_cache):
            normed = ctx.buffer("normed", (residual.shape[0], residual.shape[1]), ctx.dtype)
            self.mixer_norm.forward(residual, normed)
            self.mixer.forward(normed, residual, ctx, cache_layer, writes_cache)
            self.feed_forward.forward(normed, residual, ctx)       # the same input: the second norm is not used

    def build(d):
        rope = PartSpec("rope", {"head_dim": 64, "base": 1e4, "style": "half"})
        norm = lambda p: PartSpec("toy_layernorm", {"eps": 1e-5}, prefix=p)
        layers = tuple(LayerSpec(
            prefix=f"h.{i}.", arrangement="toy_parallel",
            mixer=PartSpec("gqa_attention", {"n_heads": 4, "n_kv_heads": 2, "head_dim": 64, "qkv_bias": True, "position": rope},
                           prefix="attn."),
            feed_forward=PartSpec("swiglu", {"intermediate_size": d["inter"]}, prefix="mlp."),
            mixer_norm=norm("ln."), feed_forward_norm=norm("unused_ln.")) for i in range(2))
        return ModelSpec(hidden_size=d["hidden"], vocab_size=d["vocab"], max_positions=256, layers=layers,
                         schedule=default_schedule(2), final_norm=norm("ln_f."),
                         embedding_name="wte.weight", head_name=None)

    register_architecture("ToyParallelLM", lambda d: d, build, replace=True)


def _plain_parallel(w, tokens, inter):
    def layernorm(x, pre):
        mean = x.mean(dim=-1, keepdim=True)
        var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
        return (x - mean) / torch.sqrt(var + 1e-5) * w[pre + "weight"] + w[pre + "bias"]
    n = len(tokens)
    h = plain_impl.embedding(w["wte.weight"], tokens)
    cos, sin = plain_impl.rope_table(64, 1e4, n)
    for i in range(2):
        pre = f"h.{i}."
        xn = layernorm(h, pre + "ln.")
        a, _ = plain_impl.attention(xn, w, pre + "attn.", n_heads=4, n_kv_heads=2, head_dim=64, cos=cos, sin=sin,
                                    rope_style="half")
        h = h + a + plain_impl.swiglu(xn, w, pre + "mlp.")
    return plain_impl.linear(layernorm(h, "ln_f."), w["wte.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_another_norm_and_another_arrangement(dtype, tmp_path):
    from rust_inference_b200.config.registry import get_architecture, unregister_architecture
    from rust_inference_b200.engine.engine import Engine
    from rust_inference_b200.engine.model import declared_tensors
    from rust_inference_b200.parts.registry import unregister
    from rust_inference_b200.weights.loader import random_tensors
    from rust_inference_b200.weights.safetensors_io import write_safetensors
    _register_parallel()
    try:
        cfg = {"architectures": ["ToyParallelLM"], "hidden": 136, "inter": 200, "vocab": 77}
        folder = str(tmp_path / "parallel")
        os.makedirs(folder)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        names = declared_tensors(get_architecture("ToyParallelLM").build_spec(cfg))
        assert "h.0.ln.bias" in names and "h.1.unused_ln.weight" in names and "ln_f.bias" in names
        write_safetensors(os.path.join(folder, "model.safetensors"), dict(random_tensors(names, 4, std=0.08, norm_std=0.2)))
        weights = oracle_weights(folder)
        eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=512)
        toks = random_tokens(70, 77, seed=3)
        want = _plain_parallel(weights, toks, 200)
        s = eng.alloc_slot()
        head = eng.step([s], [toks[:41]], "all").cpu()
        tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in toks[41:]])
        assert rel_err(torch.cat([head, tail]), want) <= (1e-4 if dtype == "float32" else 4e-2)
        eng.check_device_status()
    finally:
        unregister("norm", "toy_layernorm")
        unregister("arrangement", "toy_parallel")
        unregister_architecture("ToyParallelLM")
