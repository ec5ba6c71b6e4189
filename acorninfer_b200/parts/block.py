"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``x += mixer(norm_m(x)); x += feed_forward(norm_f(x))``
(``Qwen3Block`` in ``acorninfer/models/qwen3.py:399-410``).  The residual stream is float32;
each sum is fused into the norm that follows it, so a block takes ``(resid32, delta)``
where ``delta`` is what the previous block still has to add, and returns the same pair.
"""

from __future__ import annotations

from .base import BLOCKS, Block


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, ctx, mixer, feed_forward, norms):
        super().__init__(mixer, feed_forward, norms)
        missing = {"mixer", "feed_forward"} - set(norms)
        if missing:
            raise ValueError(f"prenorm block needs norms named 'mixer' and 'feed_forward'; missing {sorted(missing)}")

    def forward(self, resid32, delta, inputs, cache):
        h = self.norms["mixer"].add_forward(resid32, delta)
        delta = self.mixer.forward(h, inputs, cache)
        h = self.norms["feed_forward"].add_forward(resid32, delta)
        delta = self.feed_forward.forward(h, inputs)
        return resid32, delta
