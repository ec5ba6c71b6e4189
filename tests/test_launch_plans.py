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
            assert M <= 32 and splits == 2
        if M > 64:
            assert per_sm == 2


def test_gemm_plans_of_the_decode_shapes():
    # Qwen3-8B layer sizes at 8 rows: qkv, o, gate_up, down, output matrix
    assert gemm_tc_plan(8, 6144, 4096) == (4, 2)
    assert gemm_tc_plan(8, 4096, 4096) == (8, 2)
    assert gemm_tc_plan(8, 24576, 4096) == (2, 3)    # 192 tiles on 148 SMs: half tiles, three CTAs to an SM
    assert gemm_tc_plan(8, 4096, 12288) == (8, 2)
    assert gemm_tc_plan(8, 151936, 4096) == (1, 2)
