"""How a layer's parts are wired (transformer.rs:20-48)."""
from __future__ import annotations

from .base import Arrangement
from .registry import register


@register("arrangement", "pre_norm")
class PreNorm(Arrangement):
    """h1 = x + mixer(norm(x)); h2 = h1 + ff(norm(h1)): the un-normalised stream is carried
    (transformer.rs:31-47).  Roles: mixer, feed_forward, mixer_norm, feed_forward_norm."""

    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def forward(self, residual, ctx, cache_layer, writes_cache):
        normed = ctx.buffer("normed", (residual.shape[0], residual.shape[1]), ctx.dtype)
        self.mixer_norm.forward(residual, normed)
        self.mixer.forward(normed, residual, ctx, cache_layer, writes_cache)
        self.feed_forward_norm.forward(residual, normed)
        self.feed_forward.forward(normed, residual, ctx)
