"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``, no bias, every token through the
one set of matrices.  Reference: ``Qwen3MLP`` in ``acorninfer/models/qwen3.py:385-396``.
gate and up are concatenated when bound: one matrix product gives ``[tokens, 2 I]``.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, BuildContext, FeedForward, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, ctx: BuildContext, hidden_size: int, intermediate_size: int):
        self.ctx = ctx
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        return {
            "gate_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            "up_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            "down_proj.weight": TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def bind(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        dtype = g.dtype if g.dtype == u.dtype else torch.float32
        self.w_gate_up = torch.cat([g.to(dtype), u.to(dtype)], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, x, inputs):
        gu = ops.linear(x, self.w_gate_up, out_dtype=self.ctx.dtype)
        h = ops.swiglu(gu)
        return ops.linear(h, self.w_down, out_dtype=self.ctx.dtype)
