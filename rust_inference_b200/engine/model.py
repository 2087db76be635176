"""A decoder assembled from a `ModelSpec`: embedding, the scheduled layers, final norm, head.

This is the whole-stack step of the reference (transformer.rs:63-98: embedding row, the
layers in order, final RMSNorm, lm_head) for a packed batch of tokens, with the final
norm and the head run only on the rows whose logits are wanted.  It knows no
architecture: which parts a layer has and in which order layers run comes from the spec.
"""
from __future__ import annotations

import torch

from ..parts.registry import lookup
from ..parts.spec import ModelSpec, TensorSpec


def _build(category: str, part_spec, *, hidden_size, dtype, device):
    return lookup(category, part_spec.kind)(hidden_size=hidden_size, dtype=dtype, device=device,
                                            **part_spec.params)


class _Layer:
    """The parts of one layer, built for the roles its arrangement declares."""

    def __init__(self, layer_spec, *, hidden_size, dtype, device):
        self.spec = layer_spec
        arrangement = lookup("arrangement", layer_spec.arrangement)
        roles = dict(arrangement.ROLES)
        given = set(layer_spec.parts)
        unknown = sorted(given - set(roles))
        missing = sorted(set(roles) - given - set(arrangement.OPTIONAL))
        if unknown or missing:
            raise ValueError(
                f"layer {layer_spec.prefix!r}: arrangement {layer_spec.arrangement!r} has the roles {sorted(roles)}"
                + (f"; missing: {missing}" if missing else "") + (f"; not a role of it: {unknown}" if unknown else ""))
        kw = dict(hidden_size=hidden_size, dtype=dtype, device=device)
        self.parts = {role: _build(roles[role], layer_spec.parts[role], **kw) for role in roles if role in given}
        owners = [role for role in self.parts if roles[role] == "mixer"]
        if len(owners) > 1:
            raise ValueError(f"layer {layer_spec.prefix!r}: {owners} would share one cache layer; a layer has one mixer")
        self.cache_owner = self.parts[owners[0]] if owners else None
        self.block = arrangement(**self.parts)

    def cache_request(self):
        return self.cache_owner.cache_request() if self.cache_owner is not None else None

    def named_parts(self):
        for role, part in self.parts.items():
            yield self.spec.prefix + self.spec.parts[role].prefix, part


class LayerProbe:
    """The reference's debug probe (transformer.rs:80-96: min, max, mean and the first four values
    of the hidden vector after every layer and after the final norm, at position 0) for chosen rows
    of a step's packed tokens.  `stats[row]` is a list of (label, dict) in the order the layers ran:
    "L0", "L1", ... (one per schedule entry), then "FNL"."""

    def __init__(self, rows):
        self.rows = [int(r) for r in rows]
        self.stats = {r: [] for r in self.rows}

    def record(self, label: str, hidden: torch.Tensor, picked: bool = False) -> None:
        x = hidden if picked else hidden[self.rows]
        x = x.float()
        summary = torch.stack([x.amin(dim=1), x.amax(dim=1), x.sum(dim=1) / x.shape[1]], dim=1).cpu()
        first = x[:, :4].cpu()
        for i, r in enumerate(self.rows):
            self.stats[r].append((label, {"min": float(summary[i, 0]), "max": float(summary[i, 1]),
                                          "mean": float(summary[i, 2]), "first": [float(v) for v in first[i]]}))

    @staticmethod
    def format(label: str, s: dict) -> str:
        """One line in the reference's layout (transformer.rs:84-85)."""
        return (f"  [{label}] min={s['min']:9.4f} max={s['max']:9.4f} mean={s['mean']:9.4f} h0..3="
                + ",".join(f"{v:.4f}" for v in s["first"]))


class DecoderModel:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"run dtype must be float32 or bfloat16, not {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        kw = dict(hidden_size=spec.hidden_size, dtype=dtype, device=device)
        self._embedding_spec, self._head_spec = spec.embedding_part(), spec.head_part()
        self.embedding = _build("embedding", self._embedding_spec, **kw)
        self.layers = [_Layer(ls, **kw) for ls in spec.layers]
        self.head = _build("head", self._head_spec, **kw)

        # the schedule: who writes which cache layer
        seen = set()
        self.schedule = []
        self._cache_requests = [None] * spec.cache_layers()
        for entry in spec.schedule:
            if not (0 <= entry.layer < len(self.layers)):
                raise ValueError(f"schedule names layer {entry.layer}, the model has {len(self.layers)}")
            writes = entry.cache not in seen
            seen.add(entry.cache)
            request = self.layers[entry.layer].cache_request()
            if writes:
                self._cache_requests[entry.cache] = request
            elif request != self._cache_requests[entry.cache]:
                raise ValueError(
                    f"schedule: layer {entry.layer} reads cache {entry.cache}, whose owner keeps "
                    f"{self._cache_requests[entry.cache]}, not {request}")
            self.schedule.append((entry.layer, entry.cache, writes))

    # ---- tensors -----------------------------------------------------------
    def _named_parts(self):
        yield self._embedding_spec.prefix, self.embedding
        for layer in self.layers:
            yield from layer.named_parts()
        yield self._head_spec.prefix, self.head

    def declared_tensors(self) -> dict:
        out = {}
        for prefix, part in self._named_parts():
            for local, ts in part.tensor_specs().items():
                if prefix + local in out:
                    raise ValueError(f"two parts declare the tensor {prefix + local!r}")
                out[prefix + local] = ts
        return out

    def _to(self, t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        """t on the model's device in `dtype`: the copy up in the stored precision, the change of
        precision on the device (bfloat16 <-> float32 by the library's own kernel)."""
        t = t.to(device=self.device).contiguous()
        if t.dtype == dtype:
            return t
        if self.device.type == "cuda" and {t.dtype, dtype} == {torch.float32, torch.bfloat16}:
            from ..kernels import ops
            return ops.cast(t, dtype)
        return t.to(dtype)

    def _place(self, t: torch.Tensor, ts: TensorSpec) -> torch.Tensor:
        if ts.role == "matrix":
            return self._to(t, self.dtype)
        if ts.role == "vector":
            return self._to(t, torch.float32)
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
            part, local = owners[name]
            bucket = pending.setdefault(id(part), (part, {}))[1]
            bucket[local] = placed
            if len(bucket) == counts[id(part)]:
                part.set_tensors(bucket)
                del pending[id(part)]
        missing = sorted(set(declared) - got)
        if missing:
            raise KeyError(f"model is missing tensors: {', '.join(missing)}")
        if self.head.wants_tie:
            table = self.embedding.table()
            if table is None:
                raise ValueError("the head is tied to the embedding, which has no table to share")
            self.head.tie(table)                          # the same storage, no copy

    def state_dict(self) -> dict:
        """Every tensor of the model under the name the weight file gives it, as the model holds it
        on the device (matrices in the run dtype, vectors float32): what the parts packed together
        (q, k and v in one matrix) comes back apart, as views.  A tied head is not listed: it is the
        embedding.  The reference has no counterpart (it only reads, model.rs:157-203)."""
        out = {}
        for prefix, part in self._named_parts():
            for local, t in part.get_tensors().items():
                out[prefix + local] = t
        declared = self.declared_tensors()
        if set(out) != set(declared):
            raise RuntimeError("state_dict: the parts returned other tensors than they declared: "
                               f"{sorted(set(out) ^ set(declared))}")
        return {name: out[name] for name in declared}

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
        skip = set()
        if not include_embedding and not self.head.wants_tie:
            skip = {self._embedding_spec.prefix + local for local in self.embedding.tensor_specs()}
        for name, ts in self.declared_tensors().items():
            n = 1
            for d in ts.shape:
                n *= d
            if name in skip:
                continue
            total += n * (item if ts.role == "matrix" else 4)
        return total

    # ---- the step --------------------------------------------------------------
    def forward(self, ctx, cache, logits_out: torch.Tensor | None = None, probe: "LayerProbe | None" = None):
        """Run the step's tokens: the embedding part fills the float32 hidden stream, the scheduled
        layers add to it, the head part turns the wanted rows into float32 logits [wanted rows, vocab]
        (None when nothing is wanted).  `probe` (a debugging aid, never inside a captured step)
        records statistics of the hidden state after every layer."""
        residual = ctx.buffer("residual", (ctx.n_tokens, self.spec.hidden_size), torch.float32)
        self.embedding.forward(ctx, residual)
        for run, (layer, cache_index, writes) in enumerate(self.schedule):
            self.layers[layer].block.forward(residual, ctx, cache.layer(cache_index), writes)
            if probe is not None:
                probe.record(f"L{run}", residual)
        if probe is not None:
            normed = self.head.normalised(residual, torch.tensor(probe.rows, dtype=torch.int32, device=self.device))
            if normed is not None:
                probe.record("FNL", normed, picked=True)
        if ctx.n_logit_rows == 0:
            return None
        return self.head.forward(residual, ctx, logits_out)


def declared_tensors(spec: ModelSpec) -> dict:
    """Names and shapes of every tensor the model built from `spec` wants."""
    return DecoderModel(spec, dtype=torch.float32, device="cpu").declared_tensors()
