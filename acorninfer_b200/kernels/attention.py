"""Choice of the attention kernel for a step, behind one call.

The float32 engine always runs the plain kernel.  The bfloat16 engine runs the fast
kernels where they apply (single-token rows: split-K decode kernel; prompt portions:
tensor-core prefill kernel) and the plain kernel for head sizes those do not take.
"""

from __future__ import annotations

import torch

from . import ops


def paged_attention(qkv: torch.Tensor, inputs, group, cache, nq: int, nkv: int, d: int, scale: float,
                    window: int | None) -> torch.Tensor:
    """Attention of all tokens of the step; q is the head of ``qkv`` ([T, (nq + 2 nkv) d])."""
    return ops.attention_plain(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                               group.page_base, inputs.token_row, inputs.positions, inputs.num_tokens,
                               nq, nkv, d, scale, window)
