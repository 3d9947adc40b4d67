"""Arrangements of a layer's parts."""
from __future__ import annotations

from ..registry import register_block
from .base import Block


@register_block("pre_norm")
class PreNormBlock(Block):
    """hidden += mixer(norm(hidden)); hidden += feed_forward(norm(hidden))
    (crates/model-runtime/src/execute.rs:24,196-199,236)."""

    graph_safe = True

    def forward(self, hidden, ctx, cache):
        x = self.mixer_norm.forward(hidden, ctx)
        hidden = self.mixer.forward(x, ctx, cache, residual=hidden)
        x = self.feed_forward_norm.forward(hidden, ctx)
        return self.feed_forward.forward(x, ctx, residual=hidden)
