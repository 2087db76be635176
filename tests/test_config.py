"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY
from rust_inference_b200 import ConfigError, config_from_dict, load_config, registered_architectures
from rust_inference_b200.config.registry import get_architecture, register_architecture, unregister_architecture


def test_registry_maps_both_names_to_one_model():
    assert {"LlamaForCausalLM", "Qwen2ForCausalLM"} <= set(registered_architectures())
    a = get_architecture("LlamaForCausalLM")
    b = get_architecture("Qwen2ForCausalLM")
    assert a.build_spec is b.build_spec


def test_unknown_architecture_lists_registered():
    with pytest.raises(ConfigError) as e:
        config_from_dict({"architectures": ["MambaForCausalLM"], "hidden_size": 8})
    assert "MambaForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)


@pytest.mark.parametrize("name", sorted(TINY))
def test_values_come_from_config_json(name):
    d = TINY[name]
    c = config_from_dict(d)
    assert c.hidden_size == d["hidden_size"] and c.num_hidden_layers == d["num_hidden_layers"]
    assert c.num_attention_heads == d["num_attention_heads"]
    assert c.num_key_value_heads == d["num_key_value_heads"]
    assert c.intermediate_size == d["intermediate_size"] and c.vocab_size == d["vocab_size"]
    assert c.rope_theta == d["rope_theta"] and c.rms_norm_eps == d["rms_norm_eps"]
    assert c.head_dim == d.get("head_dim", d["hidden_size"] // d["num_attention_heads"])
    assert c.q_dim == c.num_attention_heads * c.head_dim and c.kv_dim == c.num_key_value_heads * c.head_dim
    # round trip through the config.json form
    assert config_from_dict(c.to_dict()) == c


def test_soft_defaults_follow_the_architecture():
    base = {"hidden_size": 64, "num_hidden_layers": 1, "num_attention_heads": 4, "intermediate_size": 32,
            "vocab_size": 10}
    llama = config_from_dict({"architectures": ["LlamaForCausalLM"], **base})
    qwen = config_from_dict({"architectures": ["Qwen2ForCausalLM"], **base})
    assert llama.rope_theta == 1e4 and qwen.rope_theta == 1e6           # model.rs:91-92
    assert llama.attention_bias is False and qwen.attention_bias is True
    assert llama.num_key_value_heads == 4                                 # model.rs:100
    assert llama.head_dim == 16                                           # model.rs:153
    assert llama.rms_norm_eps == 1e-5                                     # model.rs:86
    assert llama.max_position_embeddings == 32768                         # model.rs:103
    assert llama.tie_word_embeddings is False and llama.eos_token_ids == ()


def test_sizes_are_required():
    d = dict(TINY["A"])
    del d["intermediate_size"], d["vocab_size"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert "intermediate_size" in str(e.value) and "vocab_size" in str(e.value)


@pytest.mark.parametrize("patch, word", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 7}, "even"),
    ({"hidden_size": 130, "head_dim": None}, "multiple"),
    ({"hidden_size": -4}, "positive"),
    ({"num_hidden_layers": 2.5}, "integer"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"use_sliding_window": True, "sliding_window": 128}, "sliding"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_style": "spiral"}, "rope_style"),
    ({"rms_norm_eps": 0.0}, "positive"),
])
def test_validation_errors(patch, word):
    d = dict(TINY["A"])
    d.update(patch)
    d = {k: v for k, v in d.items() if v is not None}
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_eos_ids_int_or_list():
    d = dict(TINY["A"])
    assert config_from_dict({**d, "eos_token_id": 7}).eos_token_ids == (7,)
    assert config_from_dict({**d, "eos_token_id": [7, 9]}).eos_token_ids == (7, 9)


def test_load_config_errors(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))                       # no config.json
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY["B"]))
    assert load_config(str(tmp_path)).architecture == "Qwen2ForCausalLM"


def test_spec_is_built_layer_by_layer():
    c = config_from_dict(TINY["B"])
    spec = get_architecture(c.architecture).build_spec(c)
    assert len(spec.layers) == 3 and len(spec.schedule) == 3
    assert [e.layer for e in spec.schedule] == [0, 1, 2] and [e.cache for e in spec.schedule] == [0, 1, 2]
    layer = spec.layers[1]
    assert layer.mixer.kind == "gqa_attention" and layer.feed_forward.kind == "swiglu"
    assert layer.mixer.params["n_kv_heads"] == 2 and layer.mixer.params["qkv_bias"] is True
    assert layer.mixer.params["position"].params == {"head_dim": 128, "base": 1000000.0, "style": "interleaved"}
    assert layer.mixer_norm.params == {"eps": 1e-6}
    assert spec.head_name == "lm_head.weight"
    tied = get_architecture("LlamaForCausalLM").build_spec(config_from_dict(TINY["A"]))
    assert tied.head_name is None


def test_register_a_new_architecture():
    def parse(d):
        return d

    def build(cfg):
        return None

    register_architecture("ToyForCausalLM", parse, build)
    try:
        assert "ToyForCausalLM" in registered_architectures()
        with pytest.raises(ValueError):
            register_architecture("ToyForCausalLM", parse, build)
        assert config_from_dict({"architectures": ["ToyForCausalLM"]}) == {"architectures": ["ToyForCausalLM"]}
    finally:
        unregister_architecture("ToyForCausalLM")


def test_max_seq_len_may_shorten_the_context_but_not_lengthen_it():
    """--max-seq-len overrides the model's context length (model.rs:142-144); beyond
    max_position_embeddings the model has no positions, which is an error here."""
    from rust_inference_b200.engine.engine import resolve_max_seq_len
    assert resolve_max_seq_len(None, 2048) == 2048
    assert resolve_max_seq_len(64, 2048) == 64
    assert resolve_max_seq_len(2048, 2048) == 2048
    with pytest.raises(ValueError, match="exceeds the model's max_position_embeddings 2048"):
        resolve_max_seq_len(4096, 2048)
    with pytest.raises(ValueError, match="positive"):
        resolve_max_seq_len(0, 2048)
