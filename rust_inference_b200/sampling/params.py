"""Sampling options, with the reference's names and meanings (sampler.rs:22-48)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplerConfig:
    """The reference's `SamplerConfig` with its defaults (sampler.rs:22-48): temperature 0.8,
    top_k 40, top_p 0.95, repetition penalty 1.1 over the last 64 tokens, seed 12345.

    temperature <= 0 is greedy (sampler.rs:81-83); the penalty is applied before greedy too
    (sampler.rs:76-78).  top_k 0 (or >= vocabulary) and top_p 1.0 switch those filters off,
    repetition_penalty 1.0 switches the penalty off; `SamplerConfig.plain(...)` is
    temperature (or greedy) sampling with everything else off."""
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    repetition_penalty: float = 1.1
    repetition_window: int = 64
    seed: int = 12345

    def __post_init__(self):
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must lie in (0, 1]")
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be positive")
        if self.repetition_window < 0:
            raise ValueError("repetition_window must be >= 0")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def uses_history(self) -> bool:
        return self.repetition_penalty != 1.0 and self.repetition_window > 0

    @classmethod
    def plain(cls, temperature: float = 0.0, seed: int = 12345) -> "SamplerConfig":
        return cls(temperature=temperature, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=seed)
