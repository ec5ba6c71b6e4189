"""Choice of the attention kernel for a step, behind one call.

The float32 engine always runs the plain kernel.  The bfloat16 engine runs the split-K
decode kernel when every row of the step is a single token, the tensor-core prefill kernel
otherwise (a single-token row is then a tile of one query), and the plain kernel for head
sizes and group sizes the fast kernels do not take.
"""

from __future__ import annotations

import numpy as np
import torch

from . import ops

B200_SMS = 148          # what planning functions assume when no device is given (CPU-side tests)
_CHUNK = 64

Q_TILE = 64             # query tokens per tile of the mma.sync prefill kernel
TILE_LARGE = 128        # query tokens per tile of the tcgen05 prefill kernel
LARGE_MIN = 32          # rows shorter than this stay with the small-tile kernel


def _tiles(plan, lo: int, hi: int | None, tile: int) -> np.ndarray:
    """(row, first token within the row) of every ``tile``-token query tile of the rows that bring
    lo <= n (< hi) tokens."""
    t = [(r, q0) for r, n in enumerate(plan.row_lens) if n >= lo and (hi is None or n < hi)
         for q0 in range(0, n, tile)]
    return np.asarray(t, np.int32).reshape(-1, 2)


def _single_tokens(plan) -> np.ndarray:
    return np.asarray([int(plan.row_start[r]) for r, n in enumerate(plan.row_lens) if n == 1], np.int32)


def _large_tiles(plan) -> np.ndarray:
    """Tiles of the tcgen05 kernel, longest first: a tile's work grows with the keys before its
    last query (the row's cached length plus the tile's end), and CTAs are handed out in list
    order, so the long ones start first and the short ones fill the tail of the last wave."""
    t = _tiles(plan, LARGE_MIN, None, TILE_LARGE)
    if t.shape[0] > 1:
        keys = plan.row_pos[t[:, 0]] + np.minimum(t[:, 1] + TILE_LARGE, np.asarray(plan.row_lens, np.int32)[t[:, 0]])
        t = t[np.argsort(-keys, kind="stable")]
    return np.ascontiguousarray(t)


# The per-step arrays the attention kernels read (``Part.step_arrays``): rows of one token go to the
# decode kernel by token list, longer rows to a prefill kernel in query tiles.
STEP_ARRAYS = {
    "attention.single_tokens": _single_tokens,
    "attention.q_tiles": lambda plan: _tiles(plan, 2, None, Q_TILE),
    "attention.q_tiles_large": _large_tiles,
    "attention.q_tiles_small": lambda plan: _tiles(plan, 2, LARGE_MIN, Q_TILE),
}

sm_count = ops.device_sms


# What the split choice assumes of the decode kernel on this GPU (measured: 10 to 128 rows of 8 kv
# heads at contexts 1,024 to 16,384, 1 to 8 splits each): one CTA streams its keys and values at
# about 35 GB/s at most (three stages of 32 KB in flight), all CTAs together at the memory's 6.5
# TB/s, a wave of CTAs costs about 2 us beyond its streaming, the merge pass about 3 us.
_CTA_GBS, _HBM_GBS, _WAVE_US, _MERGE_US = 35.0, 6500.0, 2.0, 3.0


def merged_in_kernel(splits: int, limit: int) -> bool:
    """Whether a decode kernel that merges up to ``limit`` splits inside itself (a cluster) does so for
    this many: clusters of up to 8 CTAs, and of 16; sizes between (9 splits took 24 us where the
    separate merge pass took 17) are left to the merge pass."""
    return splits <= min(limit, 8) or (splits == 16 and limit >= 16)


def decode_splits(rows: int, num_kv_heads: int, key_bound: int, head_dim: int, num_sms: int = B200_SMS,
                  merge_free_upto: int = 1) -> int:
    """Splits of the key range.  ``key_bound`` bounds the keys any row reads; it changes only with
    the table stride, so a captured step keeps its grid.

    Two CTAs of the decode kernel fit on an SM: ``2 * num_sms`` (296 on a B200) run at a time, in waves.  A CTA is bound by
    its own streaming rate, a full wave by the memory.  So few (row, kv head) pairs want many
    splits (more CTAs in flight); a count just above a multiple of 296 wants splits too (a last
    wave of few long CTAs takes as long as one CTA takes alone: 40 rows of 8 kv heads, unsplit,
    take 149 us against 123 us in three splits); a count that fills its last wave well wants
    none.  The splits with the least estimated time are taken.  ``merge_free_upto``: up to this many
    splits cost no merge pass (the TMA kernel merges up to sixteen inside itself)."""
    _TARGET_CTAS = 2 * num_sms
    pairs = max(1, rows * num_kv_heads)
    most = max(1, min(-(-key_bound // _CHUNK), 32))
    pair_kb = key_bound * head_dim * 4 / 1e3                         # K and V of one pair, bfloat16, in KB
    best, best_us = 1, None
    for s in range(1, most + 1):
        kb = pair_kb / s
        alone_us = kb / _CTA_GBS                                     # KB / (GB/s) = us
        full, rest = divmod(pairs * s, _TARGET_CTAS)
        us = full * (max(alone_us, _TARGET_CTAS * kb / _HBM_GBS) + _WAVE_US)
        if rest:
            us += max(alone_us, rest * kb / _HBM_GBS) + _WAVE_US
        if not merged_in_kernel(s, merge_free_upto):
            us += _MERGE_US
        if best_us is None or us <= best_us + 1e-9:                  # equal estimates: more CTAs in flight
            best, best_us = s, us
    return best


_MERGE_FREE: dict = {}


def _merge_free(nq: int, nkv: int, d: int, P: int) -> int:
    """Splits that the decode kernel for these sizes merges itself (1: none)."""
    key = (nq, nkv, d, P)
    if key not in _MERGE_FREE:
        _MERGE_FREE[key] = (ops.lib().acorn_attention_decode_tma_merges(nq, nkv)
                            if ops.lib().acorn_attention_decode_tma_supported(nq, nkv, d, P) else 1)
    return _MERGE_FREE[key]


def paged_attention(qkv: torch.Tensor, inputs, group, cache, nq: int, nkv: int, d: int, scale: float,
                    window: int | None) -> torch.Tensor:
    """Attention of all tokens of the step; q is the head of ``qkv`` ([T, (nq + 2 nkv) d])."""
    P = cache.k_pages.shape[2]
    if qkv.dtype == torch.bfloat16:
        if inputs.plan.all_decode and ops.attention_decode_supported(nq, nkv, d) and inputs.num_tokens <= 65535:
            bound = group.block_table.shape[1] * P
            if window:
                bound = min(bound, window)
            splits = decode_splits(inputs.num_rows, nkv, bound, d, sm_count(qkv.device), _merge_free(nq, nkv, d, P))
            return ops.attention_decode(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                        group.page_base, inputs.token_row, inputs.positions, inputs.num_tokens,
                                        nq, nkv, d, scale, window, splits)
        x, hx = inputs.extra, inputs.plan.extra
        n_single = int(hx["attention.single_tokens"].size)
        if ops.attention_prefill_supported(nq, nkv, d) and (n_single == 0 or (
                ops.attention_decode_supported(nq, nkv, d) and n_single <= 65535)):
            # a mixed step: prompt portions through the prefill kernel, decoded tokens through the
            # decode kernel, both writing their rows of one output
            out = torch.empty((inputs.num_tokens, nq * d), dtype=qkv.dtype, device=qkv.device)
            if ops.attention_prefill_tc_supported(nq, nkv, d, P) and qkv.stride(0) % 8 == 0:
                # long rows on the tcgen05 kernel (tiles of 128 queries), short ones on the mma.sync kernel
                if hx["attention.q_tiles_large"].shape[0]:
                    ops.attention_prefill_tc(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                             group.page_base, inputs.row_start, inputs.row_pos, x["attention.q_tiles_large"],
                                             inputs.num_tokens, nq, nkv, d, scale, window, out=out)
                if hx["attention.q_tiles_small"].shape[0]:
                    ops.attention_prefill(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                          group.page_base, inputs.row_start, inputs.row_pos, x["attention.q_tiles_small"],
                                          inputs.num_tokens, nq, nkv, d, scale, window, out=out)
            elif hx["attention.q_tiles"].shape[0]:
                ops.attention_prefill(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                      group.page_base, inputs.row_start, inputs.row_pos, x["attention.q_tiles"],
                                      inputs.num_tokens, nq, nkv, d, scale, window, out=out)
            if n_single:
                bound = group.block_table.shape[1] * P
                if window:
                    bound = min(bound, window)
                ops.attention_decode(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                                     group.page_base, inputs.token_row, inputs.positions, inputs.num_tokens,
                                     nq, nkv, d, scale, window,
                                     decode_splits(n_single, nkv, bound, d, sm_count(qkv.device), _merge_free(nq, nkv, d, P)),
                                     token_list=x["attention.single_tokens"], out=out)
            return out
    return ops.attention_plain(qkv, qkv.stride(0), cache.k_pages, cache.v_pages, group.block_table,
                               group.page_base, inputs.token_row, inputs.positions, inputs.num_tokens,
                               nq, nkv, d, scale, window)
