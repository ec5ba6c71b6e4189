"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w`` in float32, one rounding at the end.

Reference: ``RMSNorm`` in ``acorninfer/models/qwen3.py:50-60`` (the weight multiplies in
float32 before the cast) and the fused residual-add form in ``acorninfer/ops/rmsnorm.py:15-36``.
Here the residual stream itself stays in float32, so the fused form adds the incoming
delta to it without rounding.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import NORMS, BuildContext, Norm, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, ctx: BuildContext, width: int, eps: float):
        self.ctx = ctx
        self.width = width
        self.eps = float(eps)
        self.weight32: torch.Tensor | None = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.width,), "norm")}

    def bind(self, tensors):
        # Norm weights are held in float32 whatever they were stored as (widening is exact).
        self.weight32 = tensors["weight"].to(torch.float32).contiguous()

    def as_epilogue(self, resid32):
        return ops.AddNormEpilogue(resid32, self.weight32, self.eps)

    def forward(self, x32, out=None, rows=None):
        return ops.add_rmsnorm(x32, None, self.weight32, self.eps, self.ctx.dtype, row_idx=rows, out=out)

    def add_forward(self, resid32, delta, out=None, rows=None):
        return ops.add_rmsnorm(resid32, delta, self.weight32, self.eps, self.ctx.dtype, row_idx=rows, out=out)
