"""The scheduler's decisions on the host, with a stand-in for the device step: admission,
watermark, token budget and portions, decoding, preemption of the oldest when pages run
out, recomputation, and that a scheduled step never finds the pool empty."""

import torch

from acorninfer_b200.cache.manager import CacheManager
from acorninfer_b200.engine.request import Request, RequestStatus
from acorninfer_b200.engine.scheduler import Scheduler
from acorninfer_b200.parts.base import KVNeeds
from acorninfer_b200.sampling.params import SamplingParams


def make(num_pages=16, page_size=4, max_running=4, watermark=0, budget=None, window=None):
    needs = {0: KVNeeds(1, 8, None)}
    if window:
        needs[1] = KVNeeds(1, 8, window)
    m = CacheManager(needs, {}, num_pages, page_size, max_running, dtype=torch.float32, device="cpu", allocate=False)
    return m, Scheduler(m, max_running, watermark, budget, max_step_tokens=1 << 20)


def req(i, n_prompt, max_tokens=4):
    return Request(i, list(range(1, n_prompt + 1)), SamplingParams(temperature=0.0), max_tokens, frozenset())


def run_step(m, s, decision):
    """What the engine does with a decision, without a device: write, advance, emit, retire."""
    for p in decision.portions:
        r = p.request
        assert p.start == r.cursor == r.cache.length
        m.extend(r.cache, p.start + p.length)         # must never raise: the scheduler reserved it
        m.commit(r.cache, p.start + p.length)
        r.cursor = p.start + p.length
        if p.samples:
            r.generated_ids.append(1000 + len(r.generated_ids))
            if len(r.generated_ids) >= r.max_tokens:
                r.status = RequestStatus.FINISHED
    for r in [r for r in s.running if r.is_finished]:
        s.retire(r)


def drain(m, s, limit=10000):
    steps = []
    while s.has_pending():
        d = s.schedule()
        assert d.portions or d.preempted, "an idle step is only allowed right after a preemption"
        steps.append(d)
        run_step(m, s, d)
        assert len(steps) < limit
    m.assert_balanced()
    return steps


def test_whole_prompt_then_one_token_per_step():
    m, s = make()
    r = req(0, 9, max_tokens=3)
    s.add(r)
    d = s.schedule()
    assert [(p.start, p.length, p.samples) for p in d.portions] == [(0, 9, True)] and d.admitted == [r]
    run_step(m, s, d)
    d = s.schedule()
    assert [(p.start, p.length, p.samples) for p in d.portions] == [(9, 1, True)]
    run_step(m, s, d)
    run_step(m, s, s.schedule())
    assert r.is_finished and len(r.generated_ids) == 3 and not s.has_pending()
    m.assert_balanced()


def test_budget_cuts_prompts_and_counts_decoded_tokens_first():
    m, s = make(num_pages=64, budget=8)
    a, b = req(0, 5, max_tokens=50), req(1, 20, max_tokens=2)
    s.add(a)
    run_step(m, s, s.schedule())                      # a: whole prompt (5 <= 8), first token
    s.add(b)
    d = s.schedule()
    # a decodes (1 token), b gets the remaining 7 of the budget and does not sample yet
    assert [(p.request.seq_id, p.start, p.length, p.samples) for p in d.portions] == [(0, 5, 1, True), (1, 0, 7, False)]
    run_step(m, s, d)
    d = s.schedule()
    assert [(p.request.seq_id, p.start, p.length, p.samples) for p in d.portions] == [(0, 6, 1, True), (1, 7, 7, False)]
    run_step(m, s, d)
    d = s.schedule()
    assert [(p.request.seq_id, p.start, p.length, p.samples) for p in d.portions] == [(0, 7, 1, True), (1, 14, 6, True)]
    assert all(dd.num_tokens <= 8 for dd in [d])


def test_fcfs_admission_stops_at_the_first_that_does_not_fit():
    m, s = make(num_pages=8, page_size=4, watermark=1)
    big, small = req(0, 40), req(1, 2)                # big needs 10 pages: never fits here
    s.add(big)
    s.add(small)
    d = s.schedule()
    assert d.portions == [] and s.running == []       # small may not overtake big
    s.waiting.popleft()
    d = s.schedule()
    assert [p.request.seq_id for p in d.portions] == [1]


def test_watermark_and_reserve_are_left_free():
    m, s = make(num_pages=8, page_size=4, watermark=2)
    a = req(0, 16, max_tokens=8)                      # 4 pages; its first decoded token opens a 5th
    s.add(a)
    run_step(m, s, s.schedule())
    b = req(1, 8)                                     # 2 pages: free 4 - reserve 1 (a's next page) - watermark 2 = 1 < 2
    s.add(b)
    d = s.schedule()
    assert [p.request.seq_id for p in d.portions] == [0] and d.admitted == []


def test_max_running_caps_the_batch():
    m, s = make(num_pages=64, max_running=2)
    for i in range(4):
        s.add(req(i, 3, max_tokens=2))
    d = s.schedule()
    assert len(d.portions) == 2 and len(s.waiting) == 2
    steps = [d]
    run_step(m, s, d)
    steps += drain(m, s)
    assert all(len(x.portions) <= 2 for x in steps)


def test_pages_run_out_oldest_is_preempted_and_recomputed():
    m, s = make(num_pages=6, page_size=4, max_running=3)
    a, b = req(0, 12, max_tokens=8), req(1, 12, max_tokens=3)
    s.add(a)
    s.add(b)
    run_step(m, s, s.schedule())                      # both prompts: 3 + 3 pages, pool full
    assert m.free_pages() == [0]
    d = s.schedule()                                  # both cross into a 4th page: nothing is free
    assert d.preempted == [a] and a.status is RequestStatus.WAITING and a.cursor == 0 and a.cache is None
    assert s.waiting[0] is a and a.preemptions == 1
    assert [p.request.seq_id for p in d.portions] == [1]          # not admitted again in the same step
    run_step(m, s, d)
    steps = drain(m, s)
    # a came back with prompt + its first token as one prompt, and finished with all its tokens
    again = [p for st in steps for p in st.portions if p.request is a and p.start == 0]
    assert again and again[0].length >= 13
    assert len(a.generated_ids) == 8 and len(b.generated_ids) == 3


def test_random_load_never_exhausts_in_step_and_everything_finishes():
    import random
    rng = random.Random(1)
    for budget in (None, 7):
        m, s = make(num_pages=24, page_size=4, max_running=4, watermark=1, budget=budget, window=10)
        reqs = [req(i, rng.randint(1, 30), max_tokens=rng.randint(1, 25)) for i in range(30)]
        pending = list(reqs)
        guard = 0
        while pending or s.has_pending():
            for _ in range(rng.randint(0, 2)):
                if pending:
                    s.add(pending.pop(0))
            if s.has_pending():
                d = s.schedule()
                if budget is not None:
                    assert sum(p.length for p in d.portions if p.length > 1) <= budget
                run_step(m, s, d)
            guard += 1
            assert guard < 5000
        assert all(len(r.generated_ids) == r.max_tokens for r in reqs)
        m.assert_balanced()


def test_a_request_that_runs_no_more_gives_its_pages_up_first_and_is_not_queued_again():
    """The engine runs a step ahead of the host: a request whose last allowed token is sampled but
    not yet read (pending) still holds pages.  When pages run out it is the victim although an
    older request runs, it is not queued for recomputation, and the older one keeps running."""
    m, s = make(num_pages=4, page_size=4, max_running=3)
    old, done = req(0, 8, max_tokens=8), req(1, 7, max_tokens=2)
    s.add(old)
    s.add(done)
    run_step(m, s, s.schedule())                       # both prompts: 2 + 2 pages; each has its first token
    assert m.free_pages() == [0] and s.running == [old, done]
    done.pending = 1                                   # its second and last token is sampled, the host has not read it
    assert done.exhausted and not done.is_finished
    d = s.schedule()                                   # old's next token needs a third page
    assert d.preempted == [done] and done not in s.waiting and done not in s.running and done.cache is None
    assert done.preemptions == 0 and [(p.request, p.length) for p in d.portions] == [(old, 1)]
    run_step(m, s, d)
    done.pending = 0                                   # the host reads the token: finished, holding nothing
    done.generated_ids.append(9)
    done.status = RequestStatus.FINISHED
    while s.has_pending():
        run_step(m, s, s.schedule())
    m.assert_balanced()


def test_a_finished_request_does_not_block_the_queue():
    """A preempted request that ended on the token still in flight (an eos id) must not sit at the
    head of the queue: it is dropped and the next request is admitted."""
    m, s = make(num_pages=8, page_size=4, max_running=2)
    gone, nxt = req(0, 30, max_tokens=4), req(1, 5, max_tokens=2)
    gone.status = RequestStatus.FINISHED               # needs 8 pages: it would block the queue for ever
    s.waiting.appendleft(gone)
    s.add(nxt)
    d = s.schedule()
    assert d.admitted == [nxt] and gone not in s.waiting
    while s.has_pending():
        run_step(m, s, s.schedule())
    m.assert_balanced()
