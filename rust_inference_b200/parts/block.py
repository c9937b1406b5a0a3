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


@register("arrangement", "parallel_two_norms")
class ParallelTwoNorms(Arrangement):
    """x <- x + mixer(norm_a(x)) + ff(norm_b(x)): mixer and feed-forward read the same stream, each
    through a norm of its own; both add onto the float32 stream.  A layer may have no feed-forward
    (then it has no second norm either)."""

    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}
    OPTIONAL = ("feed_forward", "feed_forward_norm")

    def forward(self, residual, ctx, cache_layer, writes_cache):
        shape = (residual.shape[0], residual.shape[1])
        normed = ctx.buffer("normed", shape, ctx.dtype)
        if self.feed_forward is not None:
            # both norms read the stream before either branch adds to it (small steps: one kernel for the two)
            normed_ff = ctx.buffer("normed_ff", shape, ctx.dtype)
            pair = getattr(self.mixer_norm, "forward_with", None)
            if pair is None or not pair(self.feed_forward_norm, residual, normed, normed_ff):
                self.mixer_norm.forward(residual, normed)
                self.feed_forward_norm.forward(residual, normed_ff)
        else:
            self.mixer_norm.forward(residual, normed)
        self.mixer.forward(normed, residual, ctx, cache_layer, writes_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(normed_ff, residual, ctx)


@register("arrangement", "parallel_shared_norm")
class ParallelSharedNorm(Arrangement):
    """x <- x + (mixer(h) + ff(h)) with h = norm(x): one norm, and mixer and feed-forward both read its
    output; both add onto the float32 stream.  A layer may have no feed-forward."""

    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm": "norm"}
    OPTIONAL = ("feed_forward",)

    def forward(self, residual, ctx, cache_layer, writes_cache):
        normed = ctx.buffer("normed", (residual.shape[0], residual.shape[1]), ctx.dtype)
        self.norm.forward(residual, normed)
        self.mixer.forward(normed, residual, ctx, cache_layer, writes_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(normed, residual, ctx)
