"""Arrangements of norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

from ..registry import BLOCKS
from .base import Block


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``h += mixer(norm(h)); h += ffn(norm(h))`` (crates/leone/src/runtime.rs:9103-9317)."""

    def forward(self, ctx, cache, hidden):
        x = self.mixer_norm.forward(ctx, hidden)
        self.mixer.forward(ctx, cache, x, hidden)
        x = self.ffn_norm.forward(ctx, hidden)
        self.feed_forward.forward(ctx, x, hidden)
