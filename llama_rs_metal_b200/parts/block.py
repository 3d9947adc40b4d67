"""Arrangements of a layer's parts."""
from __future__ import annotations

from ..registry import register_block
from .base import Block


@register_block("pre_norm")
class PreNormBlock(Block):
    """hidden += mixer(norm(hidden)); hidden += feed_forward(norm(hidden))
    (crates/model-runtime/src/execute.rs:24,196-199,236)."""

    graph_safe = True

    @property
    def folds_pending_on_entry(self) -> bool:
        return self.mixer_norm.folds_pending

    def forward(self, hidden, ctx, cache):
        after = ctx.next_folds_pending  # what comes after this block (the model says)
        x = self.mixer_norm.forward(hidden, ctx)
        # the mixer's output goes straight into the second norm: if that norm adds pending
        # partial sums itself, the mixer's last product may leave its K slices unadded
        ctx.may_defer = self.feed_forward_norm.folds_pending
        hidden = self.mixer.forward(x, ctx, cache, residual=hidden)
        ctx.may_defer = False
        x = self.feed_forward_norm.forward(hidden, ctx)
        ctx.may_defer = after
        hidden = self.feed_forward.forward(x, ctx, residual=hidden)
        ctx.may_defer = False
        return hidden
