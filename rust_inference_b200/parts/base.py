"""The interfaces a part must have.

Every part is built as `cls(hidden_size=..., dtype=..., device=..., **params)` from the
`PartSpec` that names it, declares the tensors it wants under its own (local) names,
receives them placed on the device, and then works on *packed* activations: the step's
tokens of all sequences one after another, `[T, ...]`, with no padding.  The residual
stream is float32 `[T, hidden]` in both precisions; a mixer and a feed-forward read the
normalised activations (run dtype) and ADD their result into the residual stream.

`ctx` is the step's `engine.context.StepContext`: which token belongs to which sequence,
at which position, in which cache slot; scratch buffers; the run dtype.
"""
from __future__ import annotations

import torch

from .spec import TensorSpec


class Part:
    # False if `forward` needs the host between kernels (reads a tensor back, loops in Python
    # over device data): the engine then runs decode steps eagerly instead of replaying a graph.
    graph_safe = True

    def __init__(self, *, hidden_size: int, dtype: torch.dtype, device):
        self.hidden_size = hidden_size
        self.dtype = dtype
        self.device = torch.device(device)

    def tensor_specs(self) -> dict:
        """Local tensor name -> TensorSpec."""
        return {}

    def set_tensors(self, tensors: dict) -> None:
        """Receives the declared tensors: matrices in the run dtype, vectors float32,
        tables int32, all on the device."""
        if tensors:
            raise NotImplementedError

    def get_tensors(self) -> dict:
        """The inverse of `set_tensors`: local tensor name -> tensor as it was received (views into
        whatever the part packed them into), for `DecoderModel.state_dict()`.  A part without
        tensors has nothing to return; one with tensors must say how to take its packing apart."""
        if self.tensor_specs():
            raise NotImplementedError(f"{type(self).__name__} does not un-pack its tensors (get_tensors)")
        return {}

    def prepare(self, max_positions: int) -> None:
        """Called once the largest position is known (tables and the like)."""


class Norm(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        """x float32 [*, hidden] -> out (run dtype) [R, hidden]; `rows` picks input rows."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Owns how positions enter a mixer.  For rotary encodings that is a rotation of q and
    k, which is fused with the cache write."""

    def apply_and_store(self, qkv: torch.Tensor, ctx, cache_layer, *, n_heads: int, n_kv_heads: int,
                        head_dim: int, write_kv: bool) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_request(self):
        """What one cache layer of this mixer needs: a `cache.KVRequest`, a
        `cache.StateRequest`, or None."""
        return None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_layer, writes_cache: bool) -> None:
        """residual += mix(x).  `cache_layer` is this execution's view of the cache; when
        `writes_cache` is false another layer owns it and this one only reads."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        """residual += ff(x)."""
        raise NotImplementedError


class Embedding(Part):
    """Token ids -> the float32 hidden stream."""

    def forward(self, ctx, residual: torch.Tensor) -> None:
        """Fill residual (float32 [T, hidden]) for the step's tokens (`ctx.token_ids`, `ctx.token_pos`)."""
        raise NotImplementedError

    def table(self) -> torch.Tensor | None:
        """The [vocab, hidden] matrix a tied head may share (None: nothing to share)."""
        return None


class Head(Part):
    """The hidden stream -> float32 logits, on the wanted rows only."""

    wants_tie = False         # True: the head has no matrix of its own and is given the embedding's

    def tie(self, table: torch.Tensor) -> None:
        raise NotImplementedError

    def forward(self, residual: torch.Tensor, ctx, logits_out: torch.Tensor | None = None) -> torch.Tensor:
        """float32 [ctx.n_logit_rows, vocab] for the rows `ctx.logit_rows` of the stream."""
        raise NotImplementedError

    def normalised(self, residual: torch.Tensor, rows: torch.Tensor) -> torch.Tensor | None:
        """What the head's own norm makes of the given rows, for the layer probe (None: no norm)."""
        return None

    def matrix_bytes(self) -> int:
        """Bytes of the projection matrix a step reads (shared or not)."""
        return 0


class Arrangement:
    """How a layer's parts are wired.  Built from the already-built parts, one per role.

    ROLES maps each role the arrangement has to the category its part is looked up in; a layer spec
    must give exactly these roles (those in OPTIONAL may be left out and are then None).  At most
    one role may be of category "mixer": its part owns the layer's cache."""

    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}
    OPTIONAL: tuple = ()

    def __init__(self, **parts):
        for role in self.ROLES:
            setattr(self, role, parts.get(role))

    def forward(self, residual: torch.Tensor, ctx, cache_layer, writes_cache: bool) -> None:
        raise NotImplementedError
