"""A decoder assembled from a `ModelSpec`: embedding, the scheduled layers, final norm, head.

This is the whole-stack step of the reference (transformer.rs:63-98: embedding row, the
layers in order, final RMSNorm, lm_head) for a packed batch of tokens, with the final
norm and the head run only on the rows whose logits are wanted.  It knows no
architecture: which parts a layer has and in which order layers run comes from the spec.
"""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..parts.registry import lookup
from ..parts.spec import ModelSpec, TensorSpec


def _build(category: str, part_spec, *, hidden_size, dtype, device):
    return lookup(category, part_spec.kind)(hidden_size=hidden_size, dtype=dtype, device=device,
                                            **part_spec.params)


class _Layer:
    def __init__(self, layer_spec, *, hidden_size, dtype, device):
        self.spec = layer_spec
        kw = dict(hidden_size=hidden_size, dtype=dtype, device=device)
        self.parts = {
            "mixer": _build("mixer", layer_spec.mixer, **kw),
            "feed_forward": _build("feed_forward", layer_spec.feed_forward, **kw),
            "mixer_norm": _build("norm", layer_spec.mixer_norm, **kw),
            "feed_forward_norm": _build("norm", layer_spec.feed_forward_norm, **kw),
        }
        self.block = lookup("arrangement", layer_spec.arrangement)(**self.parts)

    def named_parts(self):
        for role, part in self.parts.items():
            yield self.spec.prefix + getattr(self.spec, role).prefix, part


class DecoderModel:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"run dtype must be float32 or bfloat16, not {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        kw = dict(hidden_size=spec.hidden_size, dtype=dtype, device=device)
        self.layers = [_Layer(ls, **kw) for ls in spec.layers]
        self.final_norm = _build("norm", spec.final_norm, **kw)
        self.embedding = None
        self.head = None

        # the schedule: who writes which cache layer
        seen = set()
        self.schedule = []
        self._cache_requests = [None] * spec.cache_layers()
        for entry in spec.schedule:
            if not (0 <= entry.layer < len(self.layers)):
                raise ValueError(f"schedule names layer {entry.layer}, the model has {len(self.layers)}")
            writes = entry.cache not in seen
            seen.add(entry.cache)
            request = self.layers[entry.layer].parts["mixer"].cache_request()
            if writes:
                self._cache_requests[entry.cache] = request
            elif request != self._cache_requests[entry.cache]:
                raise ValueError(
                    f"schedule: layer {entry.layer} reads cache {entry.cache}, whose owner keeps "
                    f"{self._cache_requests[entry.cache]}, not {request}")
            self.schedule.append((entry.layer, entry.cache, writes))

    # ---- tensors -----------------------------------------------------------
    def _named_parts(self):
        for layer in self.layers:
            yield from layer.named_parts()
        yield self.spec.final_norm.prefix, self.final_norm

    def declared_tensors(self) -> dict:
        v, h = self.spec.vocab_size, self.spec.hidden_size
        out = {self.spec.embedding_name: TensorSpec((v, h))}
        for prefix, part in self._named_parts():
            for local, ts in part.tensor_specs().items():
                out[prefix + local] = ts
        if self.spec.head_name is not None:
            out[self.spec.head_name] = TensorSpec((v, h))
        return out

    def _place(self, t: torch.Tensor, ts: TensorSpec) -> torch.Tensor:
        if ts.role == "matrix":
            return t.to(device=self.device, dtype=self.dtype).contiguous()
        if ts.role == "vector":
            return t.to(device=self.device, dtype=torch.float32).contiguous()
        if ts.role == "table":
            return t.to(device=self.device, dtype=torch.int32).contiguous()
        raise ValueError(f"unknown tensor role {ts.role!r}")

    def load(self, named_tensors) -> None:
        """Takes (name, tensor) pairs covering `declared_tensors()` and hands each part its own."""
        declared = self.declared_tensors()
        owners = {}
        for prefix, part in self._named_parts():
            for local in part.tensor_specs():
                owners[prefix + local] = (part, local)
        pending: dict = {}
        counts = {id(p): len(p.tensor_specs()) for _, p in self._named_parts()}
        got = set()
        for name, t in named_tensors:
            if name not in declared:
                raise KeyError(f"tensor {name!r} is not part of the model")
            ts = declared[name]
            if tuple(t.shape) != tuple(ts.shape):
                raise ValueError(f"{name}: expected shape {list(ts.shape)}, found {list(t.shape)}")
            placed = self._place(t, ts)
            got.add(name)
            if name == self.spec.embedding_name:
                self.embedding = placed
            elif name == self.spec.head_name:
                self.head = linear.Weight(placed)
            else:
                part, local = owners[name]
                bucket = pending.setdefault(id(part), (part, {}))[1]
                bucket[local] = placed
                if len(bucket) == counts[id(part)]:
                    part.set_tensors(bucket)
                    del pending[id(part)]
        missing = sorted(set(declared) - got)
        if missing:
            raise KeyError(f"model is missing tensors: {', '.join(missing)}")
        if self.spec.head_name is None:
            self.head = linear.Weight(self.embedding)      # tied: the same storage, no copy

    def graph_safe(self) -> bool:
        """True if every part can run inside a captured CUDA graph."""
        return all(getattr(part, "graph_safe", True) for _, part in self._named_parts())

    # ---- cache and tables ----------------------------------------------------
    def cache_requests(self) -> list:
        return list(self._cache_requests)

    def prepare(self, max_positions: int) -> None:
        for _, part in self._named_parts():
            part.prepare(max_positions)

    def weight_bytes(self, include_embedding: bool = True) -> int:
        """Bytes of the weights a step reads once: every declared tensor in the precision it
        is held in (the embedding table only counts when it is also the head, or when asked)."""
        total = 0
        item = 4 if self.dtype == torch.float32 else 2
        for name, ts in self.declared_tensors().items():
            n = 1
            for d in ts.shape:
                n *= d
            if name == self.spec.embedding_name and not include_embedding and self.spec.head_name is not None:
                continue
            total += n * (item if ts.role == "matrix" else 4)
        return total

    # ---- the step --------------------------------------------------------------
    def forward(self, ctx, cache, logits_out: torch.Tensor | None = None):
        """Run the step's tokens through the scheduled layers; returns float32 logits
        [wanted rows, vocab] (None when nothing is wanted)."""
        h = self.spec.hidden_size
        residual = ctx.buffer("residual", (ctx.n_tokens, h), torch.float32)
        ops.embed_gather(self.embedding, ctx.token_ids, residual)
        for layer, cache_index, writes in self.schedule:
            self.layers[layer].block.forward(residual, ctx, cache.layer(cache_index), writes)
        if ctx.n_logit_rows == 0:
            return None
        normed = ctx.buffer("head_in", (ctx.n_logit_rows, h), self.dtype)
        self.final_norm.forward(residual, normed, rows=ctx.logit_rows)
        if logits_out is None:
            logits_out = torch.empty((ctx.n_logit_rows, self.spec.vocab_size), dtype=torch.float32,
                                     device=self.device)
        linear.logits(normed, self.head, logits_out, ctx)
        return logits_out


def declared_tensors(spec: ModelSpec) -> dict:
    """Names and shapes of every tensor the model built from `spec` wants."""
    return DecoderModel(spec, dtype=torch.float32, device="cpu").declared_tensors()
