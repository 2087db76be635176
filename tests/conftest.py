import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# ----------------------------------------------------------------------------------------
# Tiny configurations.  A and B differ in every size and option; C and D are head sizes the
# tensor-core kernels refuse (8 and 24), so they run on the generic kernels in both dtypes.
# ----------------------------------------------------------------------------------------
TINY = {
    "A": {   # Llama style: tied, no bias, explicit head_dim != hidden/heads, half pairing
        "architectures": ["LlamaForCausalLM"], "hidden_size": 128, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 176,
        "vocab_size": 264, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "attention_bias": False,
        "tie_word_embeddings": True, "max_position_embeddings": 1024, "rope_style": "half",
    },
    "B": {   # Qwen2 style: untied, biases, odd vocabulary, interleaved pairing, 3 query heads per kv head
        "architectures": ["Qwen2ForCausalLM"], "hidden_size": 192, "num_hidden_layers": 3,
        "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 328,
        "vocab_size": 391, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True,
        "tie_word_embeddings": False, "max_position_embeddings": 2048, "rope_style": "interleaved",
    },
    "C": {   # the 2-layer Llama-style config with head_dim 8
        "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2,
        "num_attention_heads": 8, "num_key_value_heads": 2, "intermediate_size": 176, "vocab_size": 256,
        "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
        "max_position_embeddings": 128,
    },
    "D": {   # the 3-layer Qwen2-style config with head_dim 24
        "architectures": ["Qwen2ForCausalLM"], "hidden_size": 144, "num_hidden_layers": 3,
        "num_attention_heads": 6, "num_key_value_heads": 3, "intermediate_size": 352, "vocab_size": 384,
        "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
        "max_position_embeddings": 256,
    },
    "E": {   # wide enough that the bf16 projections of a small step are cut over K into float32 accumulators
        "architectures": ["Qwen2ForCausalLM"], "hidden_size": 512, "num_hidden_layers": 2,
        "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 1408,
        "vocab_size": 1003, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": True,
        "tie_word_embeddings": False, "max_position_embeddings": 1024,
    },
}

# bf16 runs are compared with the plain float32 implementation holding the same bf16 weights:
# what differs is the rounding of activations, the cache and the outputs.  Observed on a B200 over all
# tests of the tiny models (2-3 layers): float32 at most 1.1e-5 (typically 1e-6); bfloat16 0.4e-2 to
# 1.7e-2, and 2.8e-2 for the head_dim-24 model drawn with std 0.1.  Rounding noise grows with depth (see
# tests/test_full_depth_gpu.py, which takes its bfloat16 bound from the plain implementation itself).
TOL = {"float32": 1e-4, "bfloat16": 4e-2}


OBSERVED: dict = {}     # test id -> largest error it computed (written out when RI_TEST_REPORT names a file)


def note_error(err: float) -> float:
    test = os.environ.get("PYTEST_CURRENT_TEST", "?").split(" ")[0]
    if not err <= OBSERVED.get(test, -1.0):
        OBSERVED[test] = err
    return err


def pytest_sessionfinish(session, exitstatus):
    path = os.environ.get("RI_TEST_REPORT")
    if path and OBSERVED:
        with open(path, "w") as f:
            for test, err in sorted(OBSERVED.items()):
                f.write(f"{err:.3e}  {test}\n")


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Per row max|a - b| / max|b|, the worst row."""
    got, want = got.float().cpu(), want.float().cpu()
    if got.ndim == 1:
        got, want = got[None], want[None]
    return note_error(float(((got - want).abs().amax(dim=1) / want.abs().amax(dim=1).clamp_min(1e-30)).max()))


class TinyModel:
    """A model folder made in a temporary place, with its weights for the plain implementation."""

    def __init__(self, folder, cfg_dict, weights):
        self.folder = folder
        self.cfg = cfg_dict            # as written to config.json
        self.weights = weights         # name -> float32 tensor (the stored values, widened)

    def plain_logits(self, tokens, **kw):
        import plain_impl
        return plain_impl.forward(self.weights, self.cfg, tokens, **kw)


NORM_STD = 0.2      # norm weights of the test models are 1 + N(0, 0.2): no two alike, none equal to one


def oracle_weights(folder, device="cpu") -> dict:
    """The stored tensors, widened to float32, read with the `safetensors` package and not with the
    library's own reader: a tensor the library mis-slices shows against the plain implementation."""
    from safetensors.torch import load_file
    return {n: t.float() for n, t in load_file(os.path.join(folder, "model.safetensors"), device=device).items()}


def make_model(tmp_path, name, *, seed=0, std=0.05, matrix_dtype=torch.bfloat16, overrides=None, norm_std=NORM_STD):
    from rust_inference_b200 import config_from_dict, write_random_model
    d = dict(TINY[name])
    if overrides:
        d.update(overrides)
    cfg = config_from_dict(d)
    folder = str(tmp_path / f"model_{name}_{seed}")
    write_random_model(folder, cfg, seed=seed, std=std, matrix_dtype=matrix_dtype, norm_std=norm_std)
    weights = oracle_weights(folder)
    with open(os.path.join(folder, "config.json")) as f:
        cfg_dict = json.load(f)
    return TinyModel(folder, cfg_dict, weights)


@pytest.fixture(scope="session")
def model_factory(tmp_path_factory):
    cache = {}

    def get(name, seed=0, std=0.05, matrix_dtype=torch.bfloat16):
        key = (name, seed, std, matrix_dtype)
        if key not in cache:
            cache[key] = make_model(tmp_path_factory.mktemp("models"), name, seed=seed, std=std,
                                    matrix_dtype=matrix_dtype)
        return cache[key]
    return get


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ----------------------------------------------------------------------------------------
# Sampling against the plain implementation
# ----------------------------------------------------------------------------------------
def oracle_generate(model, prompt, n_new, *, temperature, seed, stream, top_k=0, top_p=1.0, stop_ids=()):
    """What the plain implementation generates on its own (whole sequence recomputed for every
    token, plain_impl.sample) when it is fed the uniform numbers the sampler draws for request
    `stream`: u = rng.uniform(seed, stream, number of tokens drawn so far)."""
    import plain_impl
    from rust_inference_b200.sampling import rng
    seq, out = list(prompt), []
    for i in range(n_new):
        tok = plain_impl.sample(model.plain_logits(seq)[-1], temperature=temperature, r=rng.uniform(seed, stream, i),
                                top_k=top_k, top_p=top_p)
        if tok in stop_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out


def assert_sampled_within_band(model, prompt, tokens, *, temperature, seed, stream, band):
    """For a run whose logits carry rounding (bfloat16): every sampled token must be the one the plain
    distribution gives for its uniform number, or a neighbour whose share of the unit interval begins
    or ends within `band` of that number."""
    from rust_inference_b200.sampling import rng
    seq = list(prompt)
    for i, tok in enumerate(tokens):
        logits = model.plain_logits(seq)[-1].double()
        p = torch.softmax(logits / temperature, dim=0)
        hi = float(torch.cumsum(p, dim=0)[tok])
        lo = hi - float(p[tok])
        u = rng.uniform(seed, stream, i)
        assert lo - band <= u <= hi + band, (f"draw {i} of request {stream}: token {tok} owns [{lo:.4f}, {hi:.4f}], "
                                             f"the uniform number is {u:.4f}")
        seq.append(tok)


def top_k_agrees(got: torch.Tensor, want: torch.Tensor, k: int, tol: float) -> bool:
    """True if the k largest entries of `got` are those of `want`, wherever `want`'s order is decided
    by more than the tolerance allows to move: rows are [vocab]; gaps are relative to max|want|.
    The k-th and (k+1)-th must also be apart for the set to be decided."""
    got, want = got.float().cpu(), want.float().cpu()
    scale = float(want.abs().max())
    top = torch.sort(want, descending=True)
    vals, ids = top.values[:k + 1], top.indices[:k + 1]
    gaps = (vals[:-1] - vals[1:]) / scale
    if float(gaps.min()) <= 2 * tol:
        return True                       # undecided at this tolerance: nothing to check
    return torch.sort(got, descending=True).indices[:k].tolist() == ids[:k].tolist()
