"""Block arrangements: how a layer's parts sit around the residual stream.

"parallel_residual": x <- x + m * (Mixer(norm1(x)) + FeedForward(norm2(x))), both norms
of the same x (one pass gives both; a layer that names no second norm feeds norm1(x) to both), m a parameter of the arrangement; the two outputs
stay pending with their multiplier and the next norm folds them in, in 32-bit.

"prenorm" is the Qwen3 decoder layer, x += Mixer(norm(x)); x += FeedForward(norm(x))
(engine/model.py:294-302 of willzeng274/kernel-rush-kawk). The adds are not done
here: a branch output stays pending on the stream and the next norm, wherever it
sits (this layer, the next one, or the final norm), folds it in.
"""

from __future__ import annotations

from .base import Block, Stream, register_block


class PreNormBlock(Block):
    def forward(self, ctx, stream: Stream, cache) -> Stream:
        h = self.mixer_norm.forward(ctx, stream)
        branch = self.mixer.forward(ctx, h, cache)
        h.tensor()  # a mixer that never looked at its input still moves the stream on
        stream.branch = branch
        if self.feed_forward is None:
            return stream

        h = self.feed_forward_norm.forward(ctx, stream)
        branch = self.feed_forward.forward(ctx, h)
        h.tensor()
        stream.branch = branch
        return stream


class ParallelResidualBlock(Block):
    """Mixer and feed-forward side by side on one x. ``params``: multiplier (default 1)."""

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward, params=None):
        super().__init__(mixer_norm, mixer, feed_forward_norm, feed_forward)
        self.multiplier = float((params or {}).get("multiplier", 1.0))
        if not hasattr(mixer_norm, "forward_pair"):
            raise TypeError("a parallel layer needs a norm that gives two norms of one x (rmsnorm_wide)")

    def forward(self, ctx, stream: Stream, cache) -> Stream:
        if self.feed_forward is None:
            h1 = self.mixer_norm.forward(ctx, stream)
            stream.branch = self.mixer.forward(ctx, h1, cache)
            stream.scale = self.multiplier
            return stream
        if self.feed_forward_norm is None:  # one norm, read by both
            h = self.mixer_norm.forward(ctx, stream)
            a = self.mixer.forward(ctx, h, cache)
            b = self.feed_forward.forward(ctx, h)
            stream.branch, stream.branch2, stream.scale = a, b, self.multiplier
            return stream
        h1, h2 = self.mixer_norm.forward_pair(ctx, stream, self.feed_forward_norm)
        a = self.mixer.forward(ctx, h1, cache)
        b = self.feed_forward.forward(ctx, h2)
        stream.branch, stream.branch2, stream.scale = a, b, self.multiplier
        return stream


register_block("prenorm", PreNormBlock)
register_block("parallel_residual", ParallelResidualBlock)
