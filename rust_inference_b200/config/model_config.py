"""Typed configuration of the Llama / Qwen2 dense decoder, read from config.json.

The reference keeps ten fields in `ModelConfig` (model.rs:35-46) and fills them from
GGUF metadata with silent per-architecture defaults for missing sizes (model.rs:89-104).
Here every size is required: a missing size is an error, not a 7B default.  Only the
reference's soft defaults are kept: kv heads = heads (model.rs:100), head_dim =
hidden / heads (model.rs:153), eps 1e-5 (model.rs:86), context 32768 (model.rs:103) and
the rope base of the architecture (model.rs:91-92).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Mapping


class ConfigError(ValueError):
    """config.json is missing a key, holds a bad value or asks for something unsupported."""


_REQUIRED_SIZES = (
    "hidden_size",
    "num_hidden_layers",
    "num_attention_heads",
    "intermediate_size",
    "vocab_size",
)


@dataclass(frozen=True)
class ArchDefaults:
    """What an architecture name implies when config.json is silent."""
    rope_theta: float
    attention_bias: bool


@dataclass(frozen=True)
class DenseDecoderConfig:
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rms_norm_eps: float
    attention_bias: bool            # biases on q, k and v (attention.rs:66-76)
    tie_word_embeddings: bool       # lm_head is the embedding matrix (model.rs:221-226)
    max_position_embeddings: int
    rope_style: str = "half"        # "half" or "interleaved" (= rope.rs:92-96)
    eos_token_ids: tuple = ()
    torch_dtype: str | None = None

    # ---- derived sizes --------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    # ---- construction ---------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any], defaults: ArchDefaults) -> "DenseDecoderConfig":
        archs = d.get("architectures")
        if not archs or not isinstance(archs, (list, tuple)):
            raise ConfigError("config.json: 'architectures' must be a non-empty list")
        missing = [k for k in _REQUIRED_SIZES if k not in d or d[k] is None]
        if missing:
            raise ConfigError(f"config.json: missing required keys: {', '.join(missing)}")

        def integer(key, value):
            if isinstance(value, bool) or not isinstance(value, int):
                raise ConfigError(f"config.json: '{key}' must be an integer, found {value!r}")
            if value <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, found {value}")
            return value

        hidden = integer("hidden_size", d["hidden_size"])
        heads = integer("num_attention_heads", d["num_attention_heads"])
        kv_heads = integer("num_key_value_heads", d.get("num_key_value_heads") or heads)
        if d.get("head_dim") is not None:
            head_dim = integer("head_dim", d["head_dim"])
        else:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads "
                    f"{heads} and no head_dim is given")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {heads} is not a multiple of "
                f"num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even for rotary pairs")

        # Things the reference has no code for (README.md:217; no scaling in rope.rs).
        if d.get("use_sliding_window") and d.get("sliding_window"):
            raise ConfigError("config.json: sliding-window attention is not supported")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: rope_scaling is not supported")
        if d.get("mlp_bias"):
            raise ConfigError("config.json: mlp_bias is not supported")

        rope_style = d.get("rope_style", "half")
        if rope_style not in ("half", "interleaved"):
            raise ConfigError(f"config.json: rope_style must be 'half' or 'interleaved', found {rope_style!r}")

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(e) for e in eos)

        rope_theta = float(d["rope_theta"]) if d.get("rope_theta") is not None else defaults.rope_theta
        eps = float(d["rms_norm_eps"]) if d.get("rms_norm_eps") is not None else 1e-5
        if rope_theta <= 0 or eps <= 0:
            raise ConfigError("config.json: rope_theta and rms_norm_eps must be positive")

        bias = d.get("attention_bias")
        if bias is None:
            bias = defaults.attention_bias

        return cls(
            architecture=str(archs[0]),
            hidden_size=hidden,
            num_hidden_layers=integer("num_hidden_layers", d["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=integer("intermediate_size", d["intermediate_size"]),
            vocab_size=integer("vocab_size", d["vocab_size"]),
            rope_theta=rope_theta,
            rms_norm_eps=eps,
            attention_bias=bool(bias),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=integer(
                "max_position_embeddings", d.get("max_position_embeddings") or 32768),
            rope_style=rope_style,
            eos_token_ids=eos_ids,
            torch_dtype=d.get("torch_dtype"),
        )

    def to_dict(self) -> dict:
        """The config.json form: the architecture's own keys."""
        d = {
            "architectures": [self.architecture],
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "attention_bias": self.attention_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_style": self.rope_style,
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder {model_dir!r}")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
