"""Arrangements of norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

from ..registry import BLOCKS
from .base import Block


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``h += mixer(norm(h)); h += ffn(norm(h))`` (crates/leone/src/runtime.rs:9103-9317)."""

    chains_norms = True       # forward takes pre= and after= (see below)

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, **extra):
        if feed_forward is None or mixer_norm is None or ffn_norm is None or extra:
            raise ValueError("the pre_norm arrangement is norm, mixer, norm, feed-forward: it takes exactly those parts")
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm)

    def entry_norm(self, ctx, hidden):
        """The norm before the mixer as a DeferredNorm for the block before this one to fill,
        or None if it has to run as a kernel."""
        if getattr(self.mixer, "accepts_deferred_norm", False):
            return self.mixer_norm.defer(ctx, hidden, "mixer")
        return None

    def forward(self, ctx, cache, hidden, pre=None, after=None):
        """``pre``: this block's entry norm, already folded into the previous block's last
        product (or None); ``after``: the next block's entry norm for this block's last product
        to fold in.  Returns ``after`` if it was filled, else None."""
        x = pre if pre is not None and pre.ready else self.mixer_norm.forward(ctx, hidden)
        mid = None
        if getattr(self.mixer, "fuses_following_norm", False) and \
                getattr(self.feed_forward, "accepts_deferred_norm", False):
            mid = self.ffn_norm.defer(ctx, hidden, "ffn")
        if mid is not None:
            self.mixer.forward(ctx, cache, x, hidden, then=mid)
        else:
            self.mixer.forward(ctx, cache, x, hidden)
        x = mid if mid is not None and mid.ready else self.ffn_norm.forward(ctx, hidden)
        if after is not None and getattr(self.feed_forward, "fuses_following_norm", False):
            self.feed_forward.forward(ctx, x, hidden, then=after)
        else:
            self.feed_forward.forward(ctx, x, hidden)
        return after if after is not None and after.ready else None
