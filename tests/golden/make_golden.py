#!/usr/bin/env python3
"""Builds tests/golden/scalar_decoder.cpp with g++, runs it on the tiny configurations A and B of
tests/conftest.py with seeded random weights, and stores the logits it computes as
tests/golden/<name>.logits.f32 (float32 [tokens, vocab]) beside the token ids it was given.

    python tests/golden/make_golden.py            # rewrites the golden files

The reference itself (a Rust crate) cannot be built here; this program is a second, independent
statement of the same formulas (scalar loops, one token at a time, a cache), against which
tests/test_plain_impl.py checks the plain implementation.  The weights are not stored: they are
made again from the seed by `rust_inference_b200.weights.loader.random_tensors`."""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

CASES = {"A": dict(seed=0, n_tokens=23, token_seed=1), "B": dict(seed=2, n_tokens=31, token_seed=3)}
STD = 0.08
NORM_STD = 0.2          # norm weights 1 + N(0, 0.2): a swapped or skipped norm weight changes the logits


def tiny_weights(name):
    """(config dict, {tensor name: float32 numpy array}) of a tiny configuration with seeded weights."""
    import torch
    from conftest import TINY
    from rust_inference_b200 import config_from_dict
    from rust_inference_b200.config.registry import get_architecture
    from rust_inference_b200.engine.model import declared_tensors
    from rust_inference_b200.weights.loader import random_tensors
    cfg = config_from_dict(TINY[name])
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    tensors = dict(random_tensors(declared_tensors(spec), CASES[name]["seed"], std=STD, matrix_dtype=torch.float32,
                                  norm_std=NORM_STD))
    return cfg, {k: v.float().numpy() for k, v in tensors.items()}


def tokens_of(name, vocab):
    rng = np.random.RandomState(CASES[name]["token_seed"])
    return [int(t) for t in rng.randint(0, vocab, size=CASES[name]["n_tokens"])]


def run_scalar(binary, cfg, w, tokens, workdir):
    order = ["model.embed_tokens.weight"]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        order += [p + "input_layernorm.weight", p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight",
                  p + "self_attn.v_proj.weight"]
        if cfg.attention_bias:
            order += [p + "self_attn.q_proj.bias", p + "self_attn.k_proj.bias", p + "self_attn.v_proj.bias"]
        order += [p + "self_attn.o_proj.weight", p + "post_attention_layernorm.weight", p + "mlp.gate_proj.weight",
                  p + "mlp.up_proj.weight", p + "mlp.down_proj.weight"]
    order.append("model.norm.weight")
    if not cfg.tie_word_embeddings:
        order.append("lm_head.weight")
    assert sorted(order) == sorted(w), "the scalar program reads every tensor of the model"
    wpath, tpath, opath = (os.path.join(workdir, n) for n in ("weights.bin", "tokens.txt", "logits.bin"))
    with open(wpath, "wb") as f:
        for name in order:
            f.write(np.ascontiguousarray(w[name], dtype=np.float32).tobytes())
    with open(tpath, "w") as f:
        f.write(" ".join(str(t) for t in tokens))
    args = [binary, wpath, tpath, opath, cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads,
            cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size, repr(float(cfg.rope_theta)),
            repr(float(cfg.rms_norm_eps)), int(cfg.attention_bias), int(cfg.tie_word_embeddings),
            0 if cfg.rope_style == "half" else 1]
    subprocess.run([str(a) for a in args], check=True)
    return np.fromfile(opath, dtype=np.float32).reshape(len(tokens), cfg.vocab_size)


def build(workdir):
    binary = os.path.join(workdir, "scalar_decoder")
    subprocess.run(["g++", "-O2", "-std=c++17", "-o", binary, os.path.join(HERE, "scalar_decoder.cpp")], check=True)
    return binary


def main():
    with tempfile.TemporaryDirectory() as tmp:
        binary = build(tmp)
        for name in CASES:
            cfg, w = tiny_weights(name)
            tokens = tokens_of(name, cfg.vocab_size)
            logits = run_scalar(binary, cfg, w, tokens, tmp)
            logits.astype(np.float32).tofile(os.path.join(HERE, f"{name}.logits.f32"))
            with open(os.path.join(HERE, f"{name}.json"), "w") as f:
                json.dump({"config": name, "weights_seed": CASES[name]["seed"], "std": STD, "norm_std": NORM_STD, "tokens": tokens,
                           "shape": list(logits.shape)}, f)
            print(f"{name}: {logits.shape}, |logits| max {np.abs(logits).max():.4f}")


if __name__ == "__main__":
    main()
