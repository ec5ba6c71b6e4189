"""The step's host-side layout: validation before anything runs, and the arrays the kernels read."""

import pytest
import torch

from acorninfer_b200.cache.manager import CacheManager
from acorninfer_b200.engine.batch import BatchError, StepEntry, StepWorkspace, plan_step, validate_entries
from acorninfer_b200.engine.request import Request
from acorninfer_b200.kernels.attention import STEP_ARRAYS
from acorninfer_b200.parts.base import KVNeeds
from acorninfer_b200.sampling.params import SamplingParams


def manager(window=None):
    needs = {0: KVNeeds(2, 16, None)}
    if window:
        needs[1] = KVNeeds(2, 16, window)
    return CacheManager(needs, {}, 64, 4, 8, dtype=torch.float32, device="cpu", allocate=False)


def test_a_bad_step_is_refused_before_anything_is_held():
    m = manager()
    a, b = m.open("a"), m.open("b")
    ok = [StepEntry(a, [1, 2, 3], [2]), StepEntry(b, [4], [0])]
    validate_entries(ok, vocab_size=10)
    for bad, word in [([], "at least one"), ([StepEntry(a, [], [])], "no tokens"),
                      ([StepEntry(a, [1, 10], [])], "outside the vocabulary"),
                      ([StepEntry(a, [1, -1], [])], "outside the vocabulary"),
                      ([StepEntry(a, [1, 2], [2])], "wanted place"),
                      ([StepEntry(a, [1], []), StepEntry(a, [2], [])], "twice")]:
        with pytest.raises(BatchError, match=word):
            validate_entries(bad, vocab_size=10)
    with pytest.raises(BatchError, match="workspace holds"):
        validate_entries(ok, vocab_size=10, max_tokens=3)
    m.close(b)
    with pytest.raises(BatchError, match="closed"):
        validate_entries([StepEntry(b, [1], [])], vocab_size=10)
    assert m.free_pages() == [64]


def test_plan_of_a_mixed_step():
    m = manager(window=6)
    a, b, c = m.open("a"), m.open("b"), m.open("c")
    for rc, n in ((a, 9), (b, 70)):                  # a and b already hold tokens
        m.extend(rc, n)
        m.commit(rc, n)
    entries = [StepEntry(a, [7], [0]), StepEntry(c, list(range(40)), [39, 0]), StepEntry(b, [3, 4], [])]
    for e in entries:
        m.extend(e.cache, e.cache.length + len(e.tokens))
    plan = plan_step(entries, m, STEP_ARRAYS)
    assert plan.num_tokens == 43 and plan.num_rows == 3 and not plan.all_decode and plan.max_q_len == 40
    assert plan.token_ids.tolist() == [7] + list(range(40)) + [3, 4]
    assert plan.positions.tolist() == [9] + list(range(40)) + [70, 71]
    assert plan.token_row.tolist() == [0] + [1] * 40 + [2, 2]
    assert plan.row_start.tolist() == [0, 1, 41, 43] and plan.row_pos.tolist() == [9, 0, 70]
    assert plan.row_slot.tolist() == [a.slot, c.slot, b.slot]
    assert plan.logit_tokens.tolist() == [0, 40, 1]              # entries in order, then `want` in order
    # the arrays the attention part declared are built by its builders, not by the step layer
    x = plan.extra
    assert x["attention.single_tokens"].tolist() == [0]                   # the decoded token of a
    assert x["attention.q_tiles"].tolist() == [[1, 0], [2, 0]]            # rows with more than one token, 64 queries a tile
    assert x["attention.q_tiles_large"].tolist() == [[1, 0]] and x["attention.q_tiles_small"].tolist() == [[2, 0]]
    assert plan_step(entries, m).extra == {}                               # no part, no extra arrays
    full, win = plan.groups
    assert full.kv_len.tolist() == [10, 40, 72] and full.page_base.tolist() == [0, 0, 0]
    assert full.block_table.shape[1] >= 18 and full.block_table.shape[1] & (full.block_table.shape[1] - 1) == 0
    assert full.block_table[2, :18].tolist() == b.tables[0]
    # the windowed group has given the front pages of b back: its table starts at page_base
    assert win.page_base.tolist() == [a.page_base[1], 0, b.page_base[1]] and b.page_base[1] > 0
    assert win.block_table[2, :len(b.tables[1])].tolist() == b.tables[1]


def test_layout_depends_on_the_shape_only_and_is_aligned():
    m = manager()
    rcs = [m.open(i) for i in range(3)]
    for rc in rcs:
        m.extend(rc, 5)
        m.commit(rc, 5)

    def decode_plan(tokens):
        entries = [StepEntry(rc, [t], [0]) for rc, t in zip(rcs, tokens)]
        for e in entries:
            m.extend(e.cache, e.cache.length + 1)
        plan = plan_step(entries, m, STEP_ARRAYS)
        for e in entries:
            m.commit(e.cache, e.cache.length + 1)
        return plan

    p1, p2 = decode_plan([1, 2, 3]), decode_plan([4, 5, 6])
    l1, n1 = StepWorkspace.layout(p1)
    l2, n2 = StepWorkspace.layout(p2)
    assert l1 == l2 and n1 == n2 and p1.all_decode                # same shape, same addresses: a graph can be replayed
    assert all(off % 4 == 0 for off, _ in l1.values())            # every array starts on 16 bytes
    names = list(l1)
    assert all(l1[a][0] + l1[a][1] <= l1[b][0] for a, b in zip(names, names[1:]))   # no overlap


def test_request_token_slices():
    r = Request(0, [1, 2, 3, 4], SamplingParams(), 8, frozenset(), generated_ids=[5, 6, 7])
    for start in range(7):
        for length in range(1, 8 - start):
            assert r.tokens(start, length) == r.all_ids[start:start + length]


def test_decode_steps_are_padded_to_buckets_with_rows_that_touch_only_the_padding_page():
    from acorninfer_b200.engine.batch import decode_bucket, pad_decode_plan
    assert [decode_bucket(n) for n in (1, 8, 9, 17, 33, 64, 65, 129, 200)] == [1, 8, 10, 20, 40, 64, 80, 160, 224]
    m = CacheManager({0: KVNeeds(2, 16, None)}, {}, 64, 4, 16, dtype=torch.float32, device="cpu", allocate=False)
    rcs = [m.open(i) for i in range(5)]
    entries = []
    for i, rc in enumerate(rcs):
        m.extend(rc, 6 + i)
        m.commit(rc, 5 + i)
        entries.append(StepEntry(rc, [i + 1], [0] if i != 2 else []))
    plan = plan_step(entries, m)
    padded = pad_decode_plan(plan, m.pad_pages, m.pad_slot, STEP_ARRAYS)
    assert (plan.num_rows, plan.num_logits) == (5, 4) and (padded.num_rows, padded.num_logits) == (5, 4)
    entries.append(StepEntry(m.open(9), [7], [0]))
    m.extend(entries[-1].cache, 1)
    plan = plan_step(entries, m)                       # 6 rows, 5 wanted -> buckets 6 and 5; force a larger case
    for k in range(3):
        rc = m.open(20 + k)
        m.extend(rc, 1)
        entries.append(StepEntry(rc, [3], [0]))
    plan = plan_step(entries, m, STEP_ARRAYS)          # 9 rows -> 10, 8 wanted -> 8
    padded = pad_decode_plan(plan, m.pad_pages, m.pad_slot, STEP_ARRAYS)
    assert padded.num_rows == padded.num_tokens == 10 and padded.num_logits == 8 and padded.all_decode
    assert padded.token_ids[:9].tolist() == plan.token_ids.tolist() and padded.token_ids[9] == 0
    assert padded.positions[9] == 0 and padded.row_slot[9] == m.pad_slot == 16 and padded.row_pos[9] == 0
    g = padded.groups[0]
    assert g.block_table[9, 0] == m.pad_pages[0] == 64 and g.kv_len[9] == 1
    assert g.block_table[:9].tolist() == plan.groups[0].block_table.tolist()
    assert padded.row_start.tolist() == list(range(11)) and padded.extra["attention.single_tokens"].tolist() == list(range(10))
    assert m.free_pages()[0] + sum(len(rc.tables[0]) for rc in m.live.values()) == 64   # the padding page is outside the pool


def test_a_captured_step_finds_its_arrays_whatever_the_patch_lists_hold():
    """Every array a captured decode step reads sits at an address that follows from the graph's key:
    rows whose token ids come from the device (the patch lists) change no other array's place, for
    every row count of a bucket, and the key tells buckets and table strides apart."""
    from acorninfer_b200.engine.batch import decode_bucket, pad_decode_plan
    m = CacheManager({0: KVNeeds(2, 16, None), 1: KVNeeds(2, 16, 6)}, {}, 256, 4, 64, dtype=torch.float32,
                     device="cpu", allocate=False)
    rcs = [m.open(i) for i in range(48)]
    for rc in rcs:
        m.extend(rc, 6)
        m.commit(rc, 5)

    def padded(R, patched):
        entries = [StepEntry(rc, [1], [0], from_device=(i if i < patched else None)) for i, rc in enumerate(rcs[:R])]
        plan = pad_decode_plan(plan_step(entries, m, STEP_ARRAYS), m.pad_pages, m.pad_slot, STEP_ARRAYS)
        return plan

    by_key = {}
    for R in list(range(1, 9)) + list(range(33, 49)):
        for patched in (0, 1, R // 2, R):
            plan = padded(R, patched)
            assert plan.patch_dst.size == patched and plan.num_rows == decode_bucket(R)
            lay, total = StepWorkspace.layout(plan)
            read_by_graph = {k: v for k, v in lay.items() if not k.startswith("patch_")}
            assert all(lay[k][0] >= max(o + n for o, n in read_by_graph.values()) for k in ("patch_dst", "patch_src"))
            key = StepWorkspace.shape_key(plan)
            assert by_key.setdefault(key, read_by_graph) == read_by_graph, (R, patched)
    assert len(by_key) == 8 + 2                                  # rows 1..8, buckets 40 and 48


def test_a_step_that_cannot_be_uploaded_gives_its_pages_back():
    m = manager()
    a = m.open("a")
    m.extend(a, 9)
    m.commit(a, 6)                     # 3 pages held, 6 tokens committed (page size 4: 2 pages needed)
    m.extend(a, 30)
    assert len(a.tables[0]) == 8
    m.trim(a)
    assert len(a.tables[0]) == 2 and m.free_pages() == [62]
    m.trim(a)                          # nothing more to give
    assert len(a.tables[0]) == 2
    m.close(a)
    m.assert_balanced()


def test_a_prompt_portion_alone_is_padded_with_tokens_that_touch_only_its_own_slots_and_the_padding_page():
    """The padded plan of a one-row step: the same row, longer; the added positions continue it; table
    entries beyond the pages the request holds name the padding page; wanted places do not move."""
    from acorninfer_b200.engine.batch import pad_prefill_plan, prefill_bucket
    from acorninfer_b200.engine.batch import prefill_buckets
    assert [prefill_bucket(n) for n in (2, 31, 32, 33, 100, 512, 513, 600, 1024)] == [32, 32, 32, 64, 128, 512, 576, 640, 1024]
    assert prefill_buckets() == list(range(32, 513, 32)) + list(range(576, 1025, 64))
    P = 4
    m = CacheManager({0: KVNeeds(2, 16, None)}, {}, 64, P, 16, dtype=torch.float32, device="cpu", allocate=False)
    rc = m.open("a")
    m.extend(rc, 9)
    m.commit(rc, 9)                                      # 9 tokens held: pages 0..2, the third holding one token
    m.extend(rc, 9 + 14)                                 # the step brings 14 more: 23 tokens, six pages
    plan = plan_step([StepEntry(rc, list(range(1, 15)), [0, 13])], m, STEP_ARRAYS)
    padded = pad_prefill_plan(plan, m.pad_pages, P, STEP_ARRAYS)
    assert (padded.num_tokens, padded.num_rows, padded.num_logits) == (32, 1, 2) and not padded.all_decode
    assert padded.token_ids[:14].tolist() == list(range(1, 15)) and not padded.token_ids[14:].any()
    assert padded.positions.tolist() == list(range(9, 41)) and padded.row_start.tolist() == [0, 32]
    assert padded.logit_tokens.tolist() == plan.logit_tokens.tolist() == [0, 13]
    g, g0 = padded.groups[0], plan.groups[0]
    assert g.kv_len.tolist() == [41] and g.max_kv_len == 41
    held = len(rc.tables[0])
    assert held == 6 and g.block_table[0, :held].tolist() == g0.block_table[0, :held].tolist() == list(rc.tables[0])
    assert g.block_table[0, held:11].tolist() == [m.pad_pages[0]] * 5           # positions 24 .. 40: pages 6 .. 10
    assert g.block_table.shape[1] >= 11
    # a plan that is a bucket already, and a plan of several rows, stay as they are
    rc2 = m.open("b")
    m.extend(rc2, 32)
    full = plan_step([StepEntry(rc2, [1] * 32, [31])], m, STEP_ARRAYS)
    assert pad_prefill_plan(full, m.pad_pages, P, STEP_ARRAYS) is full
    rc3 = m.open("c")
    m.extend(rc3, 3)
    two = plan_step([StepEntry(rc2, [1] * 32, []), StepEntry(rc3, [1, 2, 3], [2])], m, STEP_ARRAYS)
    assert pad_prefill_plan(two, m.pad_pages, P, STEP_ARRAYS) is two
