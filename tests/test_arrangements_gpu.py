"""What another architecture may need of the model's assembly, shown with toy parts that are registered
from here and never become a model of anyone's:

  * a layer whose arrangement has no feed-forward (roles: mixer, mixer_norm);
  * a layer with four norms (a norm before and after the mixer and before and after the feed-forward);
  * an embedding that scales its rows and adds learned positions, and a head that caps its logits;
  * another position encoding for the attention part: a rotation of only the first half of every head,
    with its own base, written with device-side indexing into the paged cache;
  * a mixer with fixed-size state of its own that is safe to capture: its decode update reads the
    step's slots on the device, so decode steps replay a CUDA graph.

The model is built from a spec, loaded from a folder, stepped whole, token by token through captured
graphs, and in unequal batches that reuse slots, against a plain recurrence written here."""
import json
import math
import os

import pytest
import torch

import plain_impl
from conftest import TOL, oracle_weights, random_tokens, rel_err

HIDDEN, VOCAB, MAX_POS, INTER = 128, 97, 256, 144
ROTARY_DIMS, ROTARY_BASE = 32, 5000.0        # the toy position encoding rotates 32 of a head's 64 dimensions
SCALE, CAP, DECAY, EPS = 1.5, 3.0, 0.8, 1e-5
ATT = dict(n_heads=4, n_kv_heads=2, head_dim=64)


def _register():
    from rust_inference_b200.cache.sequence_cache import StateRequest
    from rust_inference_b200.config.registry import register_architecture
    from rust_inference_b200.kernels import linear, ops
    from rust_inference_b200.parts.base import Arrangement, Embedding, Head, Mixer, PositionEncoding
    from rust_inference_b200.parts.registry import lookup, register
    from rust_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, TensorSpec, default_schedule

    @register("arrangement", "toy_mixer_only", replace=True)
    class MixerOnly(Arrangement):
        """h = x + mixer(norm(x)); nothing else."""
        ROLES = {"mixer": "mixer", "mixer_norm": "norm"}

        def forward(self, residual, ctx, cache_layer, writes_cache):
            normed = ctx.buffer("normed", tuple(residual.shape), ctx.dtype)
            self.mixer_norm.forward(residual, normed)
            self.mixer.forward(normed, residual, ctx, cache_layer, writes_cache)

    @register("arrangement", "toy_sandwich", replace=True)
    class Sandwich(Arrangement):
        """h1 = x + post(mixer(pre(x))); h2 = h1 + post'(ff(pre'(h1))): four norms."""
        ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "mixer_post_norm": "norm",
                 "feed_forward_norm": "norm", "feed_forward_post_norm": "norm"}

        def _branch(self, residual, ctx, pre, post, run):
            normed = ctx.buffer("normed", tuple(residual.shape), ctx.dtype)
            pre.forward(residual, normed)
            branch = ctx.buffer("sandwich_branch", tuple(residual.shape), torch.float32)
            branch.zero_()
            run(normed, branch)                                 # parts ADD their result: into zeros here
            post.forward(branch, normed)
            residual += normed.float()

        def forward(self, residual, ctx, cache_layer, writes_cache):
            self._branch(residual, ctx, self.mixer_norm, self.mixer_post_norm,
                         lambda x, out: self.mixer.forward(x, out, ctx, cache_layer, writes_cache))
            self._branch(residual, ctx, self.feed_forward_norm, self.feed_forward_post_norm,
                         lambda x, out: self.feed_forward.forward(x, out, ctx))

    @register("position", "toy_partial_rotary", replace=True)
    class PartialRotary(PositionEncoding):
        """Rotates the first `rotary_dims` dimensions of every q and k head (pairs (i, i + rotary_dims / 2),
        angle position / base^(2i / rotary_dims)) and leaves the rest as they are; then stores k and v
        at their positions in the paged cache.  Everything is indexed on the device (token positions,
        slots, the page table), so it runs inside captured decode steps."""

        def __init__(self, *, rotary_dims, base, hidden_size, dtype, device):
            super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
            self.rd, self.base = rotary_dims, base
            self.cos = self.sin = None

        def prepare(self, max_positions):
            cos, sin = plain_impl.rope_table(self.rd, self.base, max_positions)
            self.cos, self.sin = cos.to(self.device), sin.to(self.device)

        def apply_and_store(self, qkv, ctx, cache_layer, *, n_heads, n_kv_heads, head_dim, write_kv):
            t, half = qkv.shape[0], self.rd // 2
            qd, kvd = n_heads * head_dim, n_kv_heads * head_dim
            pos = ctx.token_pos.long()
            c, s_ = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
            for lo, heads in ((0, n_heads), (qd, n_kv_heads)):
                x = qkv[:, lo:lo + heads * head_dim].view(t, heads, head_dim)
                a, b = x[..., :half].float(), x[..., half:self.rd].float()
                lo_half, hi_half = a * c - b * s_, a * s_ + b * c        # both from the old values
                x[..., :half] = lo_half.to(qkv.dtype)
                x[..., half:self.rd] = hi_half.to(qkv.dtype)
            if write_kv:
                slot = ctx.seq_slot.long()[ctx.token_seq.long()]
                page = ctx.page_table[slot, pos // ctx.page_size].long()
                off = pos % ctx.page_size
                heads = torch.arange(n_kv_heads, device=qkv.device)
                k = qkv[:, qd:qd + kvd].view(t, n_kv_heads, head_dim)
                v = qkv[:, qd + kvd:].view(t, n_kv_heads, head_dim)
                cache_layer.k[page[:, None], heads[None, :], off[:, None]] = k
                cache_layer.v[page[:, None], heads[None, :], off[:, None]] = v

    @register("embedding", "toy_scaled_positions", replace=True)
    class ScaledWithPositions(Embedding):
        """h = table[token] * scale + positions[position]."""

        def __init__(self, *, vocab_size, max_positions, scale, hidden_size, dtype, device):
            super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
            self.vocab_size, self.max_positions, self.scale = vocab_size, max_positions, scale

        def tensor_specs(self):
            return {"weight": TensorSpec((self.vocab_size, self.hidden_size)),
                    "positions": TensorSpec((self.max_positions, self.hidden_size), role="vector")}

        def set_tensors(self, tensors):
            self.weight, self.positions = tensors["weight"], tensors["positions"]

        def get_tensors(self):
            return {"weight": self.weight, "positions": self.positions}

        def forward(self, ctx, residual):
            ops.embed_gather(self.weight, ctx.token_ids, residual)
            residual.mul_(self.scale).add_(self.positions[ctx.token_pos.long()])

    @register("head", "toy_capped", replace=True)
    class Capped(Head):
        """logits = cap * tanh((W norm(h)) / cap)."""

        def __init__(self, *, vocab_size, cap, eps, hidden_size, dtype, device):
            super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
            self.vocab_size, self.cap = vocab_size, cap
            self.norm = lookup("norm", "rmsnorm")(eps=eps, hidden_size=hidden_size, dtype=dtype, device=device)

        def tensor_specs(self):
            return {"final.weight": TensorSpec((self.hidden_size,), role="vector", init="ones"),
                    "out.weight": TensorSpec((self.vocab_size, self.hidden_size))}

        def set_tensors(self, tensors):
            self.norm.set_tensors({"weight": tensors["final.weight"]})
            self.out = linear.Weight(tensors["out.weight"])

        def get_tensors(self):
            return {"final.weight": self.norm.weight, "out.weight": self.out.t}

        def forward(self, residual, ctx, logits_out=None):
            normed = ctx.buffer("head_in", (ctx.n_logit_rows, self.hidden_size), self.dtype)
            self.norm.forward(residual, normed, rows=ctx.logit_rows)
            if logits_out is None:
                logits_out = torch.empty((ctx.n_logit_rows, self.vocab_size), dtype=torch.float32, device=residual.device)
            linear.logits(normed, self.out, logits_out, ctx)
            return logits_out.div_(self.cap).tanh_().mul_(self.cap)

    @register("mixer", "toy_decay_state", replace=True)
    class DecayState(Mixer):
        """s_t = decay * s_{t-1} + x_t per sequence (float32 state [hidden] in the cache's state area);
        residual += W s_t.  A decode step updates every sequence's state with device-side indexing by
        the step's slots, so it can be captured; a step of several tokens per sequence scans them."""
        graph_safe = True

        def __init__(self, *, decay, hidden_size, dtype, device):
            super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
            self.decay = decay

        def tensor_specs(self):
            return {"out.weight": TensorSpec((self.hidden_size, self.hidden_size))}

        def set_tensors(self, tensors):
            self.w = linear.Weight(tensors["out.weight"])

        def get_tensors(self):
            return {"out.weight": self.w.t}

        def cache_request(self):
            return StateRequest((self.hidden_size,), torch.float32)

        def forward(self, x, residual, ctx, cache_layer, writes_cache):
            state = cache_layer.state                                   # [slots, hidden] float32
            if ctx.all_single:
                slots = ctx.seq_slot.long()                             # on the device: nothing here needs the host
                s = state.index_select(0, slots) * self.decay + x.float()
                if writes_cache:
                    state.index_copy_(0, slots, s)
                mixed = s
            else:
                mixed = torch.empty(x.shape, dtype=torch.float32, device=x.device)
                at = 0
                for slot, n in zip(ctx.host_slots, ctx.host_counts):
                    s = state[slot].clone()
                    for t in range(at, at + n):
                        s = s * self.decay + x[t].float()
                        mixed[t] = s
                    if writes_cache:
                        state[slot] = s
                    at += n
            linear.into_residual(mixed.to(self.dtype), self.w, residual, ctx)

    def build(d):
        norm = lambda p: PartSpec("rmsnorm", {"eps": EPS}, prefix=p)
        rope = PartSpec("rope", {"head_dim": ATT["head_dim"], "base": 1e4, "style": "half"})
        partial = PartSpec("toy_partial_rotary", {"rotary_dims": ROTARY_DIMS, "base": ROTARY_BASE})
        attn = lambda position=rope: PartSpec("gqa_attention", dict(ATT, qkv_bias=False, position=position), prefix="attn.")
        ff = PartSpec("swiglu", {"intermediate_size": INTER}, prefix="mlp.")
        layers = (
            LayerSpec("l0.", "toy_mixer_only", mixer=attn(partial), mixer_norm=norm("n1.")),
            LayerSpec("l1.", "toy_sandwich", mixer=attn(), feed_forward=ff, mixer_norm=norm("n1."),
                      mixer_post_norm=norm("n2."), feed_forward_norm=norm("n3."), feed_forward_post_norm=norm("n4.")),
            LayerSpec("l2.", "pre_norm", mixer=PartSpec("toy_decay_state", {"decay": DECAY}, prefix="state."),
                      feed_forward=ff, mixer_norm=norm("n1."), feed_forward_norm=norm("n2.")),
        )
        return ModelSpec(hidden_size=HIDDEN, vocab_size=VOCAB, max_positions=MAX_POS, layers=layers,
                         schedule=default_schedule(3),
                         embedding=PartSpec("toy_scaled_positions", {"vocab_size": VOCAB, "max_positions": MAX_POS,
                                                                     "scale": SCALE}, prefix="tok."),
                         head=PartSpec("toy_capped", {"vocab_size": VOCAB, "cap": CAP, "eps": EPS}))

    register_architecture("ToyRolesLM", lambda d: d, build, replace=True)


def _unregister():
    from rust_inference_b200.config.registry import unregister_architecture
    from rust_inference_b200.parts.registry import unregister
    for category, kind in (("arrangement", "toy_mixer_only"), ("arrangement", "toy_sandwich"),
                           ("embedding", "toy_scaled_positions"), ("head", "toy_capped"), ("mixer", "toy_decay_state"),
                           ("position", "toy_partial_rotary")):
        unregister(category, kind)
    unregister_architecture("ToyRolesLM")


def _plain_partial_rotary_attention(x, w, pre):
    """Attention whose q and k heads are rotated in their first ROTARY_DIMS dimensions only."""
    n, nh, nkv, hd = x.shape[0], ATT["n_heads"], ATT["n_kv_heads"], ATT["head_dim"]
    cos, sin = plain_impl.rope_table(ROTARY_DIMS, ROTARY_BASE, n)

    def heads(name, count):
        y = plain_impl.linear(x, w[pre + name]).view(n, count, hd)
        rot = torch.stack([plain_impl.rope_apply(y[:, h, :ROTARY_DIMS], cos, sin, "half") for h in range(count)], dim=1)
        return torch.cat([rot, y[..., ROTARY_DIMS:]], dim=-1)

    q, k = heads("q_proj.weight", nh), heads("k_proj.weight", nkv)
    v = plain_impl.linear(x, w[pre + "v_proj.weight"]).view(n, nkv, hd)
    visible = torch.ones(n, n, dtype=torch.bool).tril()
    out = torch.zeros(n, nh, hd)
    for h in range(nh):
        s = (q[:, h] @ k[:, h // (nh // nkv)].t()) * (1.0 / math.sqrt(float(hd)))
        out[:, h] = plain_impl.softmax_rows(s.masked_fill(~visible, float("-inf"))) @ v[:, h // (nh // nkv)]
    return plain_impl.linear(out.reshape(n, nh * hd), w[pre + "o_proj.weight"])


def _plain(w, toks):
    n = len(toks)
    cos, sin = plain_impl.rope_table(ATT["head_dim"], 1e4, n)
    att = lambda x, pre: plain_impl.attention(x, w, pre, cos=cos, sin=sin, rope_style="half", **ATT)[0]
    norm = lambda x, name: plain_impl.rmsnorm(x, w[name], EPS)
    h = plain_impl.embedding(w["tok.weight"], toks) * SCALE + w["tok.positions"][:n]
    h = h + _plain_partial_rotary_attention(norm(h, "l0.n1.weight"), w, "l0.attn.")       # no feed-forward; partial rotary
    h = h + norm(att(norm(h, "l1.n1.weight"), "l1.attn."), "l1.n2.weight")                # four norms
    h = h + norm(plain_impl.swiglu(norm(h, "l1.n3.weight"), w, "l1.mlp."), "l1.n4.weight")
    xn, s, mixed = norm(h, "l2.n1.weight"), torch.zeros(HIDDEN), []
    for t in range(n):                                                                    # the recurrence
        s = DECAY * s + xn[t]
        mixed.append(s)
    h = h + plain_impl.linear(torch.stack(mixed), w["l2.state.out.weight"])
    h = h + plain_impl.swiglu(norm(h, "l2.n2.weight"), w, "l2.mlp.")
    logits = plain_impl.linear(norm(h, "final.weight"), w["out.weight"])
    return CAP * torch.tanh(logits / CAP)


def test_an_arrangement_gets_exactly_its_roles():
    """No GPU: a layer spec must give the roles its arrangement declares, no more and no fewer."""
    from rust_inference_b200.engine.model import DecoderModel
    from rust_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, default_schedule
    _register()
    try:
        norm = PartSpec("rmsnorm", {"eps": EPS}, prefix="n.")
        rope = PartSpec("rope", {"head_dim": 64, "base": 1e4, "style": "half"})
        attn = PartSpec("gqa_attention", dict(ATT, qkv_bias=False, position=rope), prefix="attn.")
        ff = PartSpec("swiglu", {"intermediate_size": INTER}, prefix="mlp.")

        def model(layer):
            spec = ModelSpec(hidden_size=HIDDEN, vocab_size=VOCAB, max_positions=64, layers=(layer,),
                             schedule=default_schedule(1), final_norm=norm)
            return DecoderModel(spec, dtype=torch.float32, device="cpu")

        m = model(LayerSpec("l.", "toy_mixer_only", mixer=attn, mixer_norm=norm))
        assert sorted(m.layers[0].parts) == ["mixer", "mixer_norm"]
        assert not any("mlp" in name for name in m.declared_tensors())
        with pytest.raises(ValueError, match="not a role of it: \\['feed_forward'\\]"):
            model(LayerSpec("l.", "toy_mixer_only", mixer=attn, mixer_norm=norm, feed_forward=ff))
        with pytest.raises(ValueError, match="missing: \\['feed_forward', 'feed_forward_norm'\\]"):
            model(LayerSpec("l.", "pre_norm", mixer=attn, mixer_norm=norm))
        full = model(LayerSpec("l.", "toy_sandwich", mixer=attn, feed_forward=ff, mixer_norm=norm,
                               mixer_post_norm=PartSpec("rmsnorm", {"eps": EPS}, prefix="n2."),
                               feed_forward_norm=PartSpec("rmsnorm", {"eps": EPS}, prefix="n3."),
                               feed_forward_post_norm=PartSpec("rmsnorm", {"eps": EPS}, prefix="n4.")))
        assert sum(name.endswith("weight") and ".n" in name for name in full.declared_tensors()) == 4
        # the built-in architecture is the shorthand: a token embedding and a linear head with the final norm
        from rust_inference_b200 import config_from_dict
        from rust_inference_b200.config.registry import get_architecture
        from conftest import TINY
        cfg = config_from_dict(TINY["A"])
        dense = DecoderModel(get_architecture(cfg.architecture).build_spec(cfg), dtype=torch.float32, device="cpu")
        assert type(dense.embedding).__name__ == "TokenEmbedding" and type(dense.head).__name__ == "LinearHead"
        assert dense.head.wants_tie and "lm_head.weight" not in dense.declared_tensors()
    finally:
        _unregister()


@pytest.fixture(scope="module")
def roles_model(tmp_path_factory):
    from rust_inference_b200.config.registry import get_architecture
    from rust_inference_b200.engine.model import declared_tensors
    from rust_inference_b200.weights.loader import random_tensors
    from rust_inference_b200.weights.safetensors_io import write_safetensors
    _register()
    folder = str(tmp_path_factory.mktemp("roles") / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump({"architectures": ["ToyRolesLM"]}, f)
    names = declared_tensors(get_architecture("ToyRolesLM").build_spec({}))
    assert "tok.positions" in names and "l1.n4.weight" in names and "l0.mlp.up_proj.weight" not in names
    write_safetensors(os.path.join(folder, "model.safetensors"), dict(random_tensors(names, 6, std=0.08, norm_std=0.2)))
    yield folder, oracle_weights(folder)
    _unregister()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_roles_model_in_every_cutting_with_captured_state_updates(dtype, roles_model):
    from rust_inference_b200.cache.sequence_cache import StateRequest
    from rust_inference_b200.engine.engine import Engine
    folder, weights = roles_model
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=1024, n_slots=3)
    assert eng.use_graphs and eng.model.graph_safe()            # the state mixer does not switch graphs off
    assert isinstance(eng.model.cache_requests()[2], StateRequest)
    tol = TOL[dtype]
    toks = random_tokens(90, VOCAB, seed=5)
    want = _plain(weights, toks)
    s = eng.alloc_slot()
    assert rel_err(eng.step([s], [toks], "all"), want) <= tol   # whole
    eng.free_slot(s)
    s = eng.alloc_slot()                                        # the same slot: its state starts from zero again
    head = eng.step([s], [toks[:58]], "all").cpu()
    tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in toks[58:]])
    assert eng.decode_graph(1).graph is not None                     # the late steps replayed a captured graph
    assert rel_err(torch.cat([head, tail]), want) <= tol
    eng.free_slot(s)
    # an unequal batch; the shortest ends early, its slot is taken again by a new request while the others go on
    others = [random_tokens(n, VOCAB, seed=30 + n) for n in (7, 41)]
    seqs = [toks[:60], others[0], others[1]]
    plains = [want, _plain(weights, others[0]), _plain(weights, others[1])]
    slots = [eng.alloc_slot() for _ in seqs]
    cut = [len(q) - 5 for q in seqs]
    eng.step(slots, [q[:c] for q, c in zip(seqs, cut)], "none")
    for step in range(5):
        live = [i for i in range(3) if not (i == 1 and step >= 2)]
        out = eng.step([slots[i] for i in live], [[seqs[i][cut[i] + step]] for i in live], "last").cpu()
        for row, i in enumerate(live):
            assert rel_err(out[row], plains[i][cut[i] + step]) <= tol, (step, i)
        if step == 1:
            eng.free_slot(slots[1])
            again = eng.alloc_slot()
            assert again == slots[1]
            fresh = eng.step([again], [toks[:20]], "all")
            assert rel_err(fresh, want[:20]) <= tol             # no state left over from the sequence before
            eng.free_slot(again)
    eng.check_device_status()
    eng.cache.pager.audit()
