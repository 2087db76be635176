"""A small, whole inference library for the Llama / Qwen2 dense decoder on one B200.

    from rust_inference_b200 import Model, SamplerConfig
    model = Model.load("/path/to/folder", dtype="bfloat16")          # config.json + safetensors
    results = model.generate([[1, 2, 3], [4, 5]], max_tokens=64,
                             sampler_config=SamplerConfig.plain(temperature=0.0))

The names follow the reference where it has them: `Model::load(path, max_seq_len)`
(model.rs:136), `Model::generate(prompt, max_tokens, sampler_config, ...)` (model.rs:332),
`SamplerConfig` (sampler.rs:22-35).  Prompts are token ids: the tokenizer and the chat
template of the reference are not part of this library.
"""
from __future__ import annotations

from .config.model_config import ConfigError, DenseDecoderConfig
from .config.registry import (config_from_dict, load_config, register_architecture,
                              registered_architectures)
from .sampling.params import SamplerConfig

__all__ = ["Model", "SamplerConfig", "GenerationResult", "DenseDecoderConfig", "ConfigError",
           "config_from_dict", "load_config", "register_architecture", "registered_architectures",
           "write_random_model"]


def __getattr__(name):
    # the heavy parts (torch, the kernels) load on first use
    if name == "Model":
        from .api import Model
        return Model
    if name == "GenerationResult":
        from .engine.generate import GenerationResult
        return GenerationResult
    if name == "write_random_model":
        from .weights.loader import write_random_model
        return write_random_model
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
