"""Plain data that describes a model as layers assembled from named parts.

An architecture's builder turns its typed config into a `ModelSpec`.  Nothing here
knows an architecture: a layer names its mixer, feed-forward, norms and arrangement by
the key they are registered under (`parts.registry`) and hands each its sizes and
constants as parameters, so layers of one model may differ.  The order in which layers
run is data as well (`schedule`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name, with its sizes and constants."""
    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""          # tensor-name prefix below the layer's prefix, e.g. "self_attn."


@dataclass(frozen=True)
class LayerSpec:
    prefix: str               # tensor-name prefix of the layer, e.g. "model.layers.3."
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One layer execution.

    layer       which LayerSpec (its weights) runs;
    cache       which cache layer its mixer uses.  Entries that name the same `cache`
                share keys/values (or state): the first of them in the schedule writes
                it, the later ones only read it;
    """
    layer: int
    cache: int


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    embedding_name: str = "model.embed_tokens.weight"
    head_name: str | None = "lm_head.weight"      # None: tied to the embedding
    stop_ids: tuple = ()
    # name patterns of tensors a folder may hold although the model does not read them
    ignored_tensors: tuple = ()

    def cache_layers(self) -> int:
        return 1 + max(e.cache for e in self.schedule)


def default_schedule(n_layers: int) -> tuple:
    """Each layer once, in order, each with a cache layer of its own."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(n_layers))


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part wants from the weight file.

    role  "matrix" (kept in the run dtype), "vector" (norm weights and biases: kept in
          float32 on the device whatever they were stored as) or "table" (integers, int32);
    init  how the random-weights mode fills it: "normal", "ones" or "zeros".
    """
    shape: tuple
    role: str = "matrix"
    init: str = "normal"
