"""The Llama / Qwen2 dense decoder as a `ModelSpec` (transformer.rs, attention.rs, mlp.rs).

Every layer: pre-norm arrangement, RMSNorm(eps), grouped-query attention with rotary
position encoding(base, pairing) and optional q/k/v biases, SwiGLU(intermediate size).
`LlamaForCausalLM` and `Qwen2ForCausalLM` are the same model with different defaults
(rope base 1e4 / 1e6, model.rs:91-92; biases off / on, as their checkpoints have them,
which the reference discovers from tensor presence, model.rs:251-280).
"""
from __future__ import annotations

from ..config.model_config import ArchDefaults, DenseDecoderConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, default_schedule

_DEFAULTS = {
    "LlamaForCausalLM": ArchDefaults(rope_theta=1e4, attention_bias=False),
    "Qwen2ForCausalLM": ArchDefaults(rope_theta=1e6, attention_bias=True),
}


def build_spec(cfg: DenseDecoderConfig) -> ModelSpec:
    position = PartSpec("rope", {"head_dim": cfg.head_dim, "base": cfg.rope_theta, "style": cfg.rope_style})
    layers = []
    for i in range(cfg.num_hidden_layers):
        layers.append(LayerSpec(
            prefix=f"model.layers.{i}.",
            mixer=PartSpec("gqa_attention", {
                "n_heads": cfg.num_attention_heads, "n_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "qkv_bias": cfg.attention_bias, "position": position,
            }, prefix="self_attn."),
            feed_forward=PartSpec("swiglu", {"intermediate_size": cfg.intermediate_size}, prefix="mlp."),
            mixer_norm=PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps}, prefix="input_layernorm."),
            feed_forward_norm=PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps}, prefix="post_attention_layernorm."),
            arrangement="pre_norm",
        ))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        layers=tuple(layers),
        schedule=default_schedule(cfg.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps}, prefix="model.norm."),
        embedding_name="model.embed_tokens.weight",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        stop_ids=tuple(cfg.eos_token_ids),
        # a stored head beside tied embeddings is a copy of the embedding (the reference clones it,
        # model.rs:221-226); old exports carry the rotary frequencies, which are made from the base here
        ignored_tensors=(("lm_head.weight",) if cfg.tie_word_embeddings else ()) + ("*.rotary_emb.inv_freq",),
    )


for _name, _defaults in _DEFAULTS.items():
    register_architecture(
        _name, (lambda d, _d=_defaults: DenseDecoderConfig.from_dict(d, _d)), build_spec, replace=True)
