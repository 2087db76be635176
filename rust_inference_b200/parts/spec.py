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


class LayerSpec:
    """One layer: an arrangement (how the parts are wired) and the parts it wires, by role.

    Which roles exist is the arrangement's business: it declares the roles it needs and the
    category each belongs to (`Arrangement.ROLES`), and the model builds exactly those.  The
    built-in `pre_norm` arrangement has the roles mixer, feed_forward, mixer_norm and
    feed_forward_norm; an arrangement registered elsewhere may have none of them (a layer
    without a feed-forward, one with four norms).  Roles are given as keyword arguments:

        LayerSpec(prefix="model.layers.3.", arrangement="pre_norm", mixer=PartSpec(...), ...)
    """

    def __init__(self, prefix: str, arrangement: str = "pre_norm", parts: dict | None = None, **roles):
        self.prefix = prefix          # tensor-name prefix of the layer, e.g. "model.layers.3."
        self.arrangement = arrangement
        self.parts = dict(parts or {})
        self.parts.update(roles)
        for role, part in self.parts.items():
            if not isinstance(part, PartSpec):
                raise TypeError(f"layer {prefix!r}: role {role!r} must be a PartSpec, found {type(part).__name__}")

    def __getattr__(self, role):
        try:
            return self.__dict__["parts"][role]
        except KeyError:
            raise AttributeError(role) from None

    def __repr__(self):
        return f"LayerSpec({self.prefix!r}, {self.arrangement!r}, {self.parts!r})"


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
    """A model: what turns token ids into the hidden stream (`embedding`), the layers and the order
    they run in, and what turns the hidden stream into logits (`head`).  Embedding and head are parts
    like any other, chosen by kind with their parameters, so an embedding that adds learned positions
    or scales its rows, or a head that caps its logits, is a part registered under another kind and
    not a change to the model.

    Shorthand for the usual pair: leave `embedding` and `head` out and give `final_norm`,
    `embedding_name` and `head_name` (None: the head is tied to the embedding); they stand for the
    `token_embedding` and `linear_head` parts with those tensor names."""
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: tuple
    schedule: tuple
    final_norm: PartSpec | None = None
    embedding_name: str = "model.embed_tokens.weight"
    head_name: str | None = "lm_head.weight"      # None: tied to the embedding
    stop_ids: tuple = ()
    embedding: PartSpec | None = None
    head: PartSpec | None = None

    def embedding_part(self) -> PartSpec:
        if self.embedding is not None:
            return self.embedding
        if not self.embedding_name.endswith("weight"):
            raise ValueError(f"embedding_name {self.embedding_name!r} must end in 'weight'")
        return PartSpec("token_embedding", {"vocab_size": self.vocab_size},
                        prefix=self.embedding_name[:-len("weight")])

    def head_part(self) -> PartSpec:
        if self.head is not None:
            return self.head
        if self.final_norm is None:
            raise ValueError("ModelSpec needs a head part, or a final_norm for the usual linear head")
        if self.head_name is not None and not self.head_name.endswith("weight"):
            raise ValueError(f"head_name {self.head_name!r} must end in 'weight'")
        return PartSpec("linear_head", {
            "vocab_size": self.vocab_size, "norm": self.final_norm, "tied": self.head_name is None,
            "weight_prefix": None if self.head_name is None else self.head_name[:-len("weight")]})
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
