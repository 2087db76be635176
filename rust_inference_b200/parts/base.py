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


class Arrangement:
    """How a layer's parts are wired.  Built from the already-built parts."""

    def __init__(self, *, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, residual: torch.Tensor, ctx, cache_layer, writes_cache: bool) -> None:
        raise NotImplementedError
