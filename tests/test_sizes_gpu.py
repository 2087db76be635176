"""Configurations drawn at random from what config.json allows: head sizes in steps of 16 (and one
that is not a multiple of 16 at all), any number of heads and groups, widths and vocabularies that are
no power of two.  Every one must either run and match the plain implementation (whole, then token by
token, in 32-bit and in bfloat16) or be refused with a clear error: never a wrong result."""
import random

import pytest
import torch

from conftest import TOL, make_model, random_tokens, rel_err

pytestmark = pytest.mark.gpu


def _draw(seed):
    rng = random.Random(seed)
    head_dim = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 256, 24])
    n_kv = rng.choice([1, 2, 3, 5])
    n_rep = rng.choice([1, 2, 3, 4, 7, 17])
    heads = n_kv * n_rep
    hidden = rng.choice([72, 136, 200, 264, 328])            # multiples of 8, none a power of two
    if rng.random() < 0.25:
        hidden = rng.choice([100, 148, 252])                 # rows of the matrices are not 16-byte multiples
    return {
        "architectures": [rng.choice(["LlamaForCausalLM", "Qwen2ForCausalLM"])], "hidden_size": hidden,
        "num_hidden_layers": rng.choice([1, 2, 3]), "num_attention_heads": heads, "num_key_value_heads": n_kv,
        "head_dim": head_dim, "intermediate_size": rng.choice([88, 150, 264, 333, 520]),
        "vocab_size": rng.choice([97, 300, 515, 1001]), "rope_theta": rng.choice([1e4, 5e5, 1e6]),
        "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-5]), "attention_bias": rng.random() < 0.5,
        "tie_word_embeddings": rng.random() < 0.5, "max_position_embeddings": 512,
        "rope_style": rng.choice(["half", "interleaved"]),
    }


@pytest.mark.parametrize("seed", list(range(14)))
def test_random_configuration(seed, tmp_path):
    from rust_inference_b200.engine.engine import Engine
    overrides = _draw(seed)
    model = make_model(tmp_path, "A", seed=seed, std=0.06, overrides=overrides)
    toks = random_tokens(150, overrides["vocab_size"], seed=100 + seed)
    want = model.plain_logits(toks)
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=1024)
        s = eng.alloc_slot()
        head = eng.step([s], [toks[:130]], "all").cpu()
        tail = torch.cat([eng.step([s], [[t]], "last").cpu() for t in toks[130:]])
        eng.free_slot(s)
        assert rel_err(torch.cat([head, tail]), want) <= TOL[dtype], (dtype, overrides)
        # three sequences of unequal length in one batch
        slots = [eng.alloc_slot() for _ in range(3)]
        cut = [toks[:37], toks[:5], toks[:101]]
        got = eng.step(slots, cut, "last").cpu()
        for i, c in enumerate(cut):
            assert rel_err(got[i], want[len(c) - 1]) <= TOL[dtype], (dtype, i, overrides)
        for sl in slots:
            eng.free_slot(sl)
        eng.check_device_status()
