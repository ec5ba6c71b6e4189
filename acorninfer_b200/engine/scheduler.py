"""Continuous-batching scheduler: who runs in the next step, and with how many tokens.

Policy, after the reference's ``Scheduler`` (``acorninfer/engine/scheduler.py:15-160``):
first come first served; a request is admitted when the pages of its whole prompt fit
beside a watermark and the pages this step's running requests are about to take; prompts
are cut into portions under a token budget, at most one portion per request per step;
every running request past its prompt decodes one token every step; when the pages for
this step's decodes and portions do not fit, the *oldest* running request is preempted:
its pages are given back, it returns to the front of the waiting queue and is later
recomputed from its prompt plus what it had generated.  A request preempted in a step
is not admitted again in the same step.

Differences from the reference, all deliberate: the budget counts every token of the
step (decoded tokens first, prompt portions fill the rest; the reference's budget covers
prompt tokens only, ``:72-76``); a request that is recomputed after a preemption is cut
into portions under the budget like any prompt (the reference exempts it from the budget,
``:140-143``, and recomputes it in one piece); page arithmetic is per cache group, since
groups (all keys, a window of them) have pools of their own; and when the engine runs a
step ahead of the host, a running request whose last allowed token is already sampled is
the first to give its pages up (it runs no more, so nothing is recomputed) and is not
queued again.

The scheduler decides; it touches no device.  It calls ``manager.close`` when it preempts
and ``manager.open`` when it admits, so page counts it reads are always current.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from .request import Request, RequestStatus


@dataclass
class Portion:
    request: Request
    start: int          # index into all_ids of the first token fed
    length: int
    samples: bool       # the portion ends at the last known token: its last logits choose a token


@dataclass
class StepDecision:
    portions: list[Portion] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)
    admitted: list[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(p.length for p in self.portions)


class Scheduler:
    def __init__(self, manager: CacheManager, max_running: int = 8, watermark_blocks: int = 0,
                 chunked_budget: int | None = None, max_step_tokens: int = 8192):
        if chunked_budget is not None and chunked_budget < 1:
            raise ValueError(f"chunked_budget must be >= 1, got {chunked_budget}")
        self.manager = manager
        self.max_running = max_running
        self.watermark = watermark_blocks
        self.chunked_budget = chunked_budget
        self.max_step_tokens = max_step_tokens
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []

    def add(self, req: Request) -> None:
        self.waiting.append(req)

    def has_pending(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ helpers

    def _budget(self) -> int:
        cap = self.max_step_tokens
        return cap if self.chunked_budget is None else min(cap, self.chunked_budget)

    def _plan_running(self, budget: int) -> tuple[list[Portion], list[int], int]:
        """Portions of the running requests under ``budget`` tokens: decodes first, then
        prompt portions in admission order.  Returns (portions, pages needed per group, budget left)."""
        portions: list[Portion] = []
        need = [0] * len(self.manager.groups)
        # a request whose last allowed token is sampled (perhaps not yet read by the host) runs no more
        active = [r for r in self.running if not r.exhausted and not r.is_finished]
        prompts = []
        for r in active:
            if r.cursor == r.num_tokens - 1 and r.num_generated:
                # Decoded tokens are never starved by the budget: every running request past its
                # prompt advances each step (reference: decodes are outside the budget).
                portions.append(Portion(r, r.cursor, 1, True))
                budget -= 1
            else:
                prompts.append(r)
        for r in prompts:
            remaining = r.num_tokens - r.cursor
            length = min(remaining, max(budget, 0))
            if length <= 0:
                continue
            budget -= length
            portions.append(Portion(r, r.cursor, length, r.cursor + length == r.num_tokens))
        pages_needed = self.manager.pages_needed
        for p in portions:
            for gi, n in enumerate(pages_needed(p.request.cache, p.start + p.length)):
                need[gi] += n
        return portions, need, budget

    def _pick_victim(self) -> Request:
        """A request that will not run again (its last allowed token is sampled; the host has not
        read it yet) if there is one: its pages are of no further use.  Else the oldest."""
        for r in self.running:
            if r.exhausted:
                return r
        return self.running[0]

    def _preempt(self, victim: Request) -> None:
        self.running.remove(victim)
        self.manager.close(victim.cache)
        victim.cache = None
        victim.cursor = 0
        if victim.exhausted:
            return              # it only waits for its last token to be read; nothing to recompute
        victim.status = RequestStatus.WAITING
        victim.preemptions += 1
        self.waiting.appendleft(victim)

    # ------------------------------------------------------------------ the decision

    def schedule(self) -> StepDecision:
        decision = StepDecision()
        # A preempted request may have ended on the token that was still on its way to the host
        # when it was queued again: it has nothing left to run.
        if any(r.is_finished for r in self.waiting):
            self.waiting = deque(r for r in self.waiting if not r.is_finished)
        # 1. what the running requests need this step; preempt the oldest until it fits
        while True:
            portions, need, budget_left = self._plan_running(self._budget())
            free = self.manager.free_pages()
            if all(n <= f for n, f in zip(need, free)) or not self.running:
                break
            victim = self._pick_victim()
            self._preempt(victim)
            decision.preempted.append(victim)
        reserve = need
        barred = {r.seq_id for r in decision.preempted}
        # 2. admission, first come first served
        pending = [0] * len(self.manager.groups)
        while self.waiting and len(self.running) < self.max_running:
            cand = self.waiting[0]
            if cand.seq_id in barred:
                break
            length = min(cand.num_tokens, max(budget_left, 0))
            if length <= 0:
                break
            whole = self.manager.peak_pages(cand.num_tokens, self.chunked_budget)
            free = self.manager.free_pages()
            if any(f - p - r - self.watermark < w for f, p, r, w in zip(free, pending, reserve, whole)):
                break
            if self.manager.slots.num_free < 1:
                break
            self.waiting.popleft()
            budget_left -= length
            for gi, w in enumerate(whole):
                pending[gi] += w
            cand.cache = self.manager.open(cand.seq_id)
            cand.status = RequestStatus.RUNNING
            cand.cursor = 0
            self.running.append(cand)
            decision.admitted.append(cand)
            portions.append(Portion(cand, 0, length, length == cand.num_tokens))
        decision.portions = portions
        return decision

    def retire(self, req: Request) -> None:
        """A finished request leaves: its pages and slot go back."""
        if req in self.running:
            self.running.remove(req)
        if req.cache is not None:
            self.manager.close(req.cache)
            req.cache = None
