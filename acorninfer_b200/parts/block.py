"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``x += mixer(norm_m(x)); x += feed_forward(norm_f(x))``
(``Qwen3Block`` in ``acorninfer/models/qwen3.py:399-410``).  The residual stream is float32;
each sum is fused into the norm that follows it, so a block takes ``(resid32, delta)``
where ``delta`` is what the previous block still has to add, and returns the same pair.
"""

from __future__ import annotations

from ..kernels import ops
from .base import BLOCKS, Block


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, ctx, mixer, feed_forward, norms):
        super().__init__(mixer, feed_forward, norms)
        missing = {"mixer", "feed_forward"} - set(norms)
        if missing:
            raise ValueError(f"prenorm block needs norms named 'mixer' and 'feed_forward'; missing {sorted(missing)}")

    def _fuses(self, num_rows):
        return (self.mixer.supports_epilogue and self.feed_forward.supports_epilogue
                and self.mixer.fusable(num_rows) and self.feed_forward.fusable(num_rows))

    def first_norm(self, num_rows):
        return self.norms["mixer"] if self._fuses(num_rows) else None

    def forward(self, resid32, delta, inputs, cache, next_norm=None):
        # With few rows on the tensor-core path, each residual sum and the norm after it are done
        # by the product before them (no kernel of their own); otherwise by the fused norm kernel.
        fuse = self._fuses(inputs.num_tokens)
        h = delta if isinstance(delta, ops.NormedRows) else self.norms["mixer"].add_forward(resid32, delta)
        ep = self.norms["feed_forward"].as_epilogue(resid32) if fuse else None
        if ep is not None:
            h = self.mixer.forward(h, inputs, cache, epilogue=ep)
        else:
            # a part that can, adds its result to the residual stream itself (delta None)
            if self.mixer.adds_residual:
                delta = self.mixer.forward(h, inputs, cache, residual32=resid32)
            else:
                delta = self.mixer.forward(h, inputs, cache)
            h = self.norms["feed_forward"].add_forward(resid32, delta)
        ep = next_norm.as_epilogue(resid32) if (fuse and next_norm is not None) else None
        if ep is not None:
            return resid32, self.feed_forward.forward(h, inputs, epilogue=ep)
        if self.feed_forward.adds_residual:
            return resid32, self.feed_forward.forward(h, inputs, residual32=resid32)
        return resid32, self.feed_forward.forward(h, inputs)
