"""Choice of the attention kernel for a step, behind one call.

The float32 engine always runs the plain kernel.  The bfloat16 engine runs the split-K
decode kernel when every row of the step is a single token, the tensor-core prefill kernel
otherwise (a single-token row is then a tile of one query), and the plain kernel for head
sizes and group sizes the fast kernels do not take.
"""

from __future__ import annotations

import torch

from . import ops

NUM_SMS = 148
_TARGET_CTAS = NUM_SMS * 2
_CHUNK = 64


def decode_splits(rows: int, num_kv_heads: int, key_bound: int) -> int:
    """Splits of the key range so that rows * kv heads * splits CTAs fill the GPU in one wave
    (two CTAs of the decode kernel fit on an SM), never more CTAs than that.  ``key_bound``
    bounds the keys any row reads; it changes only with the table stride, so a captured step
    keeps its grid."""
    ctas = max(1, rows * num_kv_heads)
    return max(1, min(_TARGET_CTAS // ctas, -(-key_bound // _CHUNK), 32))


def paged_attention(qkv: torch.Tensor, inputs, group, cache, nq: int, nkv: int, d: int, scale: float,
                    window: int | None) -> torch.Tensor:
    """Attention of all tokens of the step; q is the head of ``qkv`` ([T, (nq + 2 nkv) d])."""
    P = cache.k_pages.shape[2]
    if qkv.dtype == torch.bfloat16:
        if inputs.plan.all_decode and ops.attention_decode_supported(nq, nkv, d) and inputs.num_tokens <= 65535:
            bound = group.block_table.shape[1] * P
            if window:
                bound = min(bound, window)
            splits = decode_splits(inputs.num_rows, nkv, bound)
            return ops.attention_decode(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                        group.page_base, inputs.token_row, inputs.positions, inputs.num_tokens,
                                        nq, nkv, d, scale, window, splits)
        n_single = int(inputs.plan.single_tokens.size)
        if ops.attention_prefill_supported(nq, nkv, d) and (n_single == 0 or (
                ops.attention_decode_supported(nq, nkv, d) and n_single <= 65535)):
            # a mixed step: prompt portions through the prefill kernel, decoded tokens through the
            # decode kernel, both writing their rows of one output
            out = torch.empty((inputs.num_tokens, nq * d), dtype=qkv.dtype, device=qkv.device)
            if ops.attention_prefill_tc_supported(nq, nkv, d, P) and qkv.stride(0) % 8 == 0:
                # long rows on the tcgen05 kernel (tiles of 128 queries), short ones on the mma.sync kernel
                if inputs.q_tiles_large.shape[0]:
                    ops.attention_prefill_tc(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                             group.page_base, inputs.row_start, inputs.row_pos, inputs.q_tiles_large,
                                             inputs.num_tokens, nq, nkv, d, scale, window, out=out)
                if inputs.q_tiles_small.shape[0]:
                    ops.attention_prefill(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                          group.page_base, inputs.row_start, inputs.row_pos, inputs.q_tiles_small,
                                          inputs.num_tokens, nq, nkv, d, scale, window, out=out)
            elif inputs.q_tiles.shape[0]:
                ops.attention_prefill(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                      group.page_base, inputs.row_start, inputs.row_pos, inputs.q_tiles,
                                      inputs.num_tokens, nq, nkv, d, scale, window, out=out)
            if n_single:
                bound = group.block_table.shape[1] * P
                if window:
                    bound = min(bound, window)
                ops.attention_decode(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                     group.page_base, inputs.token_row, inputs.positions, inputs.num_tokens,
                                     nq, nkv, d, scale, window, decode_splits(n_single, nkv, bound),
                                     token_list=inputs.single_tokens, out=out)
            return out
    return ops.attention_plain(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                               group.page_base, inputs.token_row, inputs.positions, inputs.num_tokens,
                               nq, nkv, d, scale, window)
