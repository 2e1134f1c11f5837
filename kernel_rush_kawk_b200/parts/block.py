"""Block arrangements: how a layer's parts sit around the residual stream.

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

        h = self.feed_forward_norm.forward(ctx, stream)
        branch = self.feed_forward.forward(ctx, h)
        h.tensor()
        stream.branch = branch
        return stream


register_block("prenorm", PreNormBlock)
