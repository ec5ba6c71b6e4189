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
    supports_epilogue = True
    adds_residual = True

    def __init__(self, ctx: BuildContext, hidden_size: int, intermediate_size: int):
        self.ctx = ctx
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.w_gate_up = self.w_down = None
        # gate and up rows are stored in blocks: `block` gate rows, then the `block` up rows of the
        # same outputs.  64 puts a gate/up pair of blocks in every 128-row tile of the tcgen05
        # product, whose epilogue can then apply SwiGLU itself.
        self.block = 64 if intermediate_size % 64 == 0 else intermediate_size

    def tensor_specs(self):
        return {
            "gate_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            "up_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            "down_proj.weight": TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def bind(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        dtype = g.dtype if g.dtype == u.dtype else torch.float32
        b, I, H = self.block, self.intermediate_size, self.hidden_size
        self.w_gate_up = torch.stack([g.to(dtype).view(I // b, b, H), u.to(dtype).view(I // b, b, H)], dim=1) \
            .reshape(2 * I, H).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def fusable(self, num_rows):
        widths = (2 * self.intermediate_size, self.hidden_size)                 # of the gate/up product and of the down product
        return (ops.fused_rows_ok(num_rows, self.ctx.dtype, widths, ops.device_sms(self.ctx.device))
                and self.w_gate_up.dtype == torch.bfloat16
                and self.w_down.dtype == torch.bfloat16 and self.hidden_size % 8 == 0
                and self.intermediate_size % 8 == 0)

    def _gate_up_fuses(self, num_rows):
        """The gate/up product alone on the paired kernel with SwiGLU as its epilogue: it is the widest
        product of a layer, so its tiles fill the device from far fewer rows than the whole layer needs
        (about 360 rows at Qwen3-8B widths), and the stand-alone SwiGLU kernel with its round trip is
        spared.  Measured: a gain from 384 rows on at hidden size 4,096 (a loss at 300 rows, where the
        second token tile is nearly empty); none at hidden size 1,024, where a tile's 16 k-steps are too
        few to hide its epilogue."""
        return (self.ctx.dtype == torch.bfloat16 and self.w_gate_up.dtype == torch.bfloat16 and self.hidden_size % 8 == 0
                and self.hidden_size >= ops.GEMM_PAIR_ALONE_MIN_K
                and ops.pair_rows_ok(num_rows, 2 * self.intermediate_size, ops.device_sms(self.ctx.device),
                                     ops.GEMM_PAIR_MIN_FILL_ALONE, ops.GEMM_PAIR_ALONE_MAX_ROWS))

    def forward(self, x, inputs, epilogue=None, residual32=None):
        rows = x.x.shape[0] if isinstance(x, ops.NormedRows) else x.shape[0]
        if self.block == 64 and (self.fusable(rows) or self._gate_up_fuses(rows)):
            h = ops.linear(x, self.w_gate_up, out_dtype=self.ctx.dtype, swiglu=True)
        else:
            gu = ops.linear(x, self.w_gate_up, out_dtype=self.ctx.dtype)
            h = ops.swiglu(gu, block=self.block)
        return ops.linear(h, self.w_down, out_dtype=self.ctx.dtype, epilogue=epilogue,
                          residual32=residual32 if epilogue is None else None)
