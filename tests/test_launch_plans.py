"""The choices made on the host before a launch (splits of decode attention, splits and occupancy of
the tcgen05 product) as pure functions: bounds that the kernels rely on, for any sizes."""

import random

from acorninfer_b200.kernels.attention import decode_splits
from acorninfer_b200.kernels.ops import gemm_tc_plan, gemm_tc_splits


def test_decode_splits_stay_within_what_the_kernels_take():
    rng = random.Random(0)
    for _ in range(2000):
        rows, nkv = rng.randint(1, 4096), rng.choice([1, 2, 3, 4, 5, 8, 16, 32])
        bound = rng.choice([1, 16, 63, 64, 65, 1000, 4096, 40000, 1 << 20])
        s = decode_splits(rows, nkv, bound, rng.choice([16, 64, 128, 256]))
        assert 1 <= s <= 32
        assert s <= max(1, -(-bound // 64))          # never more splits than chunks of 64 keys


def test_decode_splits_follow_the_measured_cases():
    # few pairs: many CTAs in flight; a count just above a multiple of 296: shorter CTAs; a well
    # filled last wave: no split
    assert decode_splits(1, 8, 4096, 128) >= 16
    assert decode_splits(8, 8, 4096, 128) == 4
    assert decode_splits(32, 8, 4096, 128) == 1 and decode_splits(64, 8, 4096, 128) == 1 and decode_splits(96, 8, 4096, 128) == 1
    assert decode_splits(40, 8, 4096, 128) > 1 and decode_splits(20, 8, 4096, 128) > 1 and decode_splits(80, 8, 4096, 128) > 1
    assert decode_splits(8, 8, 48, 128) == 1              # a single chunk cannot be split
    # the estimate is in bytes: a smaller head size makes a pair's keys cheaper, which never asks for more splits
    assert decode_splits(8, 8, 4096, 32) <= decode_splits(8, 8, 4096, 128)


def test_gemm_plans_are_valid_for_any_shape():
    rng = random.Random(1)
    for _ in range(3000):
        M, N, K = rng.randint(1, 300), rng.randint(1, 200000), 8 * rng.randint(1, 4096)
        splits, per_sm = gemm_tc_plan(M, N, K)
        assert splits in (1, 2, 4, 8) and per_sm in (2, 3)
        assert gemm_tc_splits(M, N, K) == splits
        if splits > 1:
            assert -(-K // 64) // splits >= 4        # every split keeps at least four steps of K
        if per_sm == 3:
            assert M <= 64 and splits == 2       # three short rings to an SM: tiles of up to 64 tokens
        if M > 64:
            assert per_sm == 2


def test_gemm_plans_of_the_decode_shapes():
    # Qwen3-8B layer sizes at 8 rows: qkv, o, gate_up, down, output matrix
    assert gemm_tc_plan(8, 6144, 4096) == (4, 2)
    assert gemm_tc_plan(8, 4096, 4096) == (8, 2)
    assert gemm_tc_plan(8, 24576, 4096) == (2, 3)    # 192 tiles on 148 SMs: half tiles, three CTAs to an SM
    assert gemm_tc_plan(8, 4096, 12288) == (8, 2)
    assert gemm_tc_plan(8, 151936, 4096) == (1, 2)


def test_paired_kernel_is_asked_for_where_its_tiles_fill_the_device():
    """256 x 256 tiles in rounds of one tile to a pair of SMs: 74 pairs on 148 SMs."""
    from acorninfer_b200.kernels.ops import fused_rows_ok, pair_rows_ok
    import torch
    assert pair_rows_ok(2048, 4096)            # 128 tiles: two rounds, 0.86 full
    assert not pair_rows_ok(1536, 4096)        # 96 tiles: two rounds, 0.65 full
    assert not pair_rows_ok(200, 4096)         # below one tile of rows
    assert not pair_rows_ok(2048, 1024, max_rows=8192) and pair_rows_ok(4608, 1024, max_rows=8192)    # a narrow model needs more rows: 32 tiles, 72 tiles on 74 pairs
    assert not pair_rows_ok(1800, 4096)        # eight token tiles, the last one a fifth full: 0.76
    # the widest product taken alone needs less: gate/up of 24,576 columns from about 360 rows on
    assert pair_rows_ok(384, 24576, min_fill=0.6) and not pair_rows_ok(300, 24576, min_fill=0.6)
    assert not pair_rows_ok(257, 24576, min_fill=0.6)     # the second token tile holds one row
    assert pair_rows_ok(3072, 4096) and not pair_rows_ok(4096, 4096)       # the longest steps: not every product (the power cap)
    assert pair_rows_ok(4096, 24576, min_fill=0.6, max_rows=8192) and not pair_rows_ok(12288, 24576, min_fill=0.6, max_rows=8192)
    assert not pair_rows_ok(2048, 1024)        # 32 tiles on 74 pairs
    assert pair_rows_ok(2048, 4096, num_sms=64) == (128 / (4 * 32) >= 0.8)
    # the one-CTA kernel's range is independent of the width; between the two ranges nothing is fused
    assert fused_rows_ok(8, torch.bfloat16) and fused_rows_ok(32, torch.bfloat16, 4096)
    assert not fused_rows_ok(33, torch.bfloat16, 4096) and not fused_rows_ok(1536, torch.bfloat16, 4096)
    assert fused_rows_ok(2048, torch.bfloat16, 4096) and not fused_rows_ok(2048, torch.bfloat16)
    # every product of the part has to fill the device: at 1,024 rows the q/k/v product of 6,144 columns does not
    assert fused_rows_ok(1024, torch.bfloat16, 4096) and not fused_rows_ok(1024, torch.bfloat16, (6144, 4096))
    assert fused_rows_ok(2048, torch.bfloat16, (6144, 4096)) and fused_rows_ok(2048, torch.bfloat16, (24576, 4096))
    assert not fused_rows_ok(2048, torch.float32, 4096)
