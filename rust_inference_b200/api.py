"""The Python entry point: load a model folder, generate from token ids."""
from __future__ import annotations

from .engine.engine import Engine, resolve_max_seq_len
from .engine.generate import GenerationResult, Generator
from .sampling.params import SamplerConfig
from .sampling.sampler import Sampler


class Model:
    """`Model.load` and `Model.generate`, as the reference names them (model.rs:136, :332)."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.config = getattr(engine, "config", None)
        self.last_stats: dict = {}

    @classmethod
    def load(cls, path: str, max_seq_len: int | None = None, *, dtype: str = "bfloat16",
             device: str = "cuda", max_tokens_in_cache: int | None = None, n_slots: int | None = None) -> "Model":
        """path: a folder with config.json and model.safetensors (or shards with an index).
        max_seq_len overrides the model's context length, as `--max-seq-len` does in the
        reference (model.rs:142-144): it caps the cache and the rotary table.
        max_tokens_in_cache: positions all live sequences may hold together (default: 8 sequences
        of max_seq_len, at most 65,536 positions)."""
        from .config.registry import load_spec
        seq = resolve_max_seq_len(max_seq_len, load_spec(path)[1].max_positions)
        if max_tokens_in_cache is None:
            max_tokens_in_cache = min(8 * seq, max(seq, 65536))
        return cls(Engine.from_pretrained(path, dtype=dtype, device=device, max_tokens=max_tokens_in_cache,
                                          max_seq_len=seq, n_slots=n_slots))

    @classmethod
    def random(cls, config, *, seed: int = 0, std: float = 0.02, norm_std: float = 0.0, dtype: str = "bfloat16",
               device: str = "cuda", max_seq_len: int | None = None, max_tokens_in_cache: int = 65536,
               n_slots: int | None = None) -> "Model":
        """A model with random weights made on the device from a typed config and a seed: matrices and
        biases N(0, std), norm weights 1 + N(0, norm_std)."""
        return cls(Engine.from_random(config, seed=seed, std=std, norm_std=norm_std, dtype=dtype, device=device,
                                      max_tokens=max_tokens_in_cache, max_seq_len=max_seq_len, n_slots=n_slots))

    def memory(self) -> dict:
        """Bytes the model holds on the device and what a decode step has to read of them: the weights
        (every declared tensor once), the weights a step reads (the embedding table only when it is also
        the head), the cache as allocated, and the cache bytes one position of one sequence adds."""
        eng = self.engine
        item = 4 if eng.dtype.itemsize == 4 else 2
        per_position = 0
        for req in eng.model.cache_requests():
            if req is not None and hasattr(req, "n_kv_heads"):
                per_position += 2 * req.n_kv_heads * req.head_dim * item
        return {"weight_bytes": eng.model.weight_bytes(), "weight_bytes_per_step": eng.model.weight_bytes(False),
                "cache_bytes": eng.cache.bytes(), "cache_bytes_per_position": per_position}

    def state_dict(self) -> dict:
        """name -> tensor for every tensor of the model, under the weight file's names, as held on the
        device (matrices in the run dtype, norm weights and biases float32; packed matrices as views
        of their parts).  Handing these to a plain implementation gives it the very numbers the
        engine computes with, without a folder on disk."""
        return self.engine.model.state_dict()

    def save_safetensors(self, folder: str) -> str:
        """Write the model as a folder (config.json, model.safetensors) that `Model.load` reads back."""
        import json
        import os
        from .weights.safetensors_io import write_safetensors
        if self.config is None:
            raise RuntimeError("save_safetensors: the model was built without a typed configuration")
        os.makedirs(folder, exist_ok=True)
        tensors = {name: t.detach().to("cpu") for name, t in self.state_dict().items()}
        write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
        with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
            json.dump(self.config.to_dict(), f, indent=2)
        return folder

    def logits(self, tokens, want="all", layer_stats: list | None = None):
        """float32 logits [wanted, vocab] of one list of token ids run whole, as one step of the
        engine (the reference computes them for every position, transformer.rs:89-97).  `want`:
        "all", "last", or a list of positions among the tokens.  The sequence's slot is given
        back afterwards.  `layer_stats`: a list that receives (label, {min, max, mean, first}) of the
        hidden vector at position 0 after every layer and after the final norm, which the reference
        prints in debug builds (transformer.rs:80-96)."""
        from .engine.model import LayerProbe
        probe = LayerProbe([0]) if layer_stats is not None else None
        slot = self.engine.alloc_slot()
        try:
            out = self.engine.step([slot], [list(tokens)], want if isinstance(want, str) else [list(want)], probe=probe)
        finally:
            self.engine.free_slot(slot)
        if probe is not None:
            layer_stats.extend(probe.stats[0])
        return out

    def generate(self, prompts, max_tokens: int = 512, sampler_config: SamplerConfig | None = None,
                 stop_ids=None, max_batch: int | None = None, record_step_times: bool = False) -> list:
        """prompts: a list of token-id lists (or one list of ints).  Returns one
        `GenerationResult` per prompt; `last_stats` then holds the call's counts (steps, prompt and
        generated tokens, seconds, tokens per second, bytes copied up and down).  stop_ids defaults to the model's eos ids
        (config.json `eos_token_id`); a sampled stop id ends its sequence and is not returned
        (model.rs:383-387).  Defaults follow the reference: max_tokens 512 (main.rs:65),
        `SamplerConfig()` (sampler.rs:37-48)."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        batch = [list(prompts)] if single else [list(p) for p in prompts]
        cfg = sampler_config or SamplerConfig()
        if stop_ids is None:
            stop_ids = self.engine.model.spec.stop_ids
        sampler = Sampler(cfg, self.engine.device)
        gen = Generator(self.engine, sampler, stop_ids=stop_ids, max_batch=max_batch)
        if record_step_times:
            gen.step_times = []
        import time
        h2d0 = self.engine.h2d_bytes + self.engine.cache.h2d_bytes
        t0 = time.perf_counter()
        results = gen.generate(batch, max_tokens)
        seconds = time.perf_counter() - t0
        # everything that went up from pinned host memory: the steps' arrays (prompts among them), new
        # page-table entries, the sampler's per-row arrays; and the sampled tokens that came down
        h2d = self.engine.h2d_bytes + self.engine.cache.h2d_bytes - h2d0 + sampler.h2d_bytes
        n_out = sum(len(r.tokens) for r in results)
        self.last_stats = {"steps": gen.steps, "h2d_bytes": h2d, "d2h_bytes": gen.d2h_bytes,
                           "step_times": gen.step_times, "seconds": seconds,
                           "prompt_tokens": sum(len(p) for p in batch), "generated_tokens": n_out,
                           "tokens_per_second": n_out / seconds if seconds > 0 else 0.0}
        return results[0] if single else results
