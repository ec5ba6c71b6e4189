"""The engine: request life cycle and the step loop above the step function.

``submit`` -> repeated ``step`` -> tokens.  A step asks the scheduler who runs, feeds all
of it to the :class:`ModelRunner` as ONE batch (prompt portions beside decoded tokens),
samples one token for every row that reached its last known token, records eos/length,
and retires what finished.  Interface and meanings after the reference's ``Engine``
(``acorninfer/engine/engine.py:133-378``): ``submit(prompt_ids, sampling, max_tokens=,
eos_ids=) -> seq_id``, ``step() -> [TokenOutput]``, ``has_pending()``, ``drop(seq_id)``,
``seqs[seq_id]``, ``assert_balanced()``.

When pages run out: the scheduler preempts the oldest running request and recomputes it
later (see scheduler).  A request that can never run because it alone needs more pages
than the pool has (its prompt is checked at submit; its growth is not known then) is
finished with ``stop_reason = "capacity"`` instead of waiting for ever.
"""

from __future__ import annotations

import time
from dataclasses import dataclass

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .request import Request, RequestStatus
from .runner import ModelRunner
from .scheduler import Scheduler


@dataclass
class _Inflight:
    """A launched step whose sampled ids the host has not read: who sampled, and the ids on the device."""

    samplers: list
    sampled: object


@dataclass
class TokenOutput:
    seq_id: int
    token_id: int
    finished: bool
    stop_reason: str | None = None


class Engine:
    def __init__(self, runner: ModelRunner, *, max_running: int = 8, watermark_blocks: int = 8,
                 chunked_budget: int | None = None, default_eos_ids=None, lookahead: bool = True):
        self.runner = runner
        self.manager = runner.manager
        if any(watermark_blocks >= t for t in self.manager.total_pages()):
            raise ValueError(f"watermark_blocks ({watermark_blocks}) must be < num_blocks ({self.manager.num_pages})")
        self.scheduler = Scheduler(self.manager, max_running, watermark_blocks, chunked_budget,
                                   runner.max_step_tokens)
        self.sampler = Sampler(runner.device)
        cfg_eos = getattr(runner.config, "eos_token_id", ())
        self.default_eos_ids = frozenset(default_eos_ids if default_eos_ids is not None else cfg_eos)
        self.seqs: dict[int, Request] = {}
        self.lookahead = lookahead
        self._inflight: _Inflight | None = None
        self._next_id = 0
        self.steps = 0
        self.host_seconds = 0.0        # time spent deciding and launching (not waiting for results), over all steps
        self.rows_launched = 0         # rows of all launched steps

    @classmethod
    def from_config(cls, cfg: EngineConfig) -> "Engine":
        runner = ModelRunner.from_model_dir(
            cfg.model_dir, dtype=cfg.dtype, device=cfg.device, num_blocks=cfg.num_blocks, page_size=cfg.page_size,
            max_requests=cfg.max_running, max_step_tokens=cfg.max_step_tokens, decode_graph=cfg.decode_graph)
        return cls(runner, max_running=cfg.max_running, watermark_blocks=cfg.watermark_blocks,
                   chunked_budget=cfg.chunked_budget)

    # ------------------------------------------------------------------ requests

    def submit(self, prompt_ids: list[int], sampling: SamplingParams | None = None, *, max_tokens: int,
               eos_ids=None) -> int:
        if not prompt_ids:
            raise ValueError("prompt_ids must be non-empty")
        if max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        for t in prompt_ids:
            if not (0 <= int(t) < self.runner.vocab_size):
                raise ValueError(f"token id {t} outside the vocabulary (0..{self.runner.vocab_size - 1})")
        need = self.manager.peak_pages(len(prompt_ids), self.scheduler.chunked_budget)
        for n, total in zip(need, self.manager.total_pages()):
            if n > total - self.scheduler.watermark:
                raise ValueError(
                    f"prompt needs {n} cache pages, the schedulable capacity is {total - self.scheduler.watermark} "
                    f"({total} pages - watermark); it could never be admitted")
        req = Request(self._next_id, [int(t) for t in prompt_ids], sampling or SamplingParams(temperature=0.0),
                      max_tokens, frozenset(eos_ids) if eos_ids is not None else self.default_eos_ids)
        self._next_id += 1
        self.seqs[req.seq_id] = req
        self.scheduler.add(req)
        return req.seq_id

    def drop(self, seq_id: int) -> None:
        req = self.seqs.get(seq_id)
        if req is not None and not req.is_finished:
            raise ValueError(f"seq {seq_id} is still pending; cannot drop")
        self.seqs.pop(seq_id, None)

    def abort(self, seq_id: int) -> None:
        """Ends a pending request now (``stop_reason = "abort"``); what it holds goes back."""
        req = self.seqs.get(seq_id)
        if req is None or req.is_finished:
            return
        if req in self.scheduler.waiting:
            self.scheduler.waiting.remove(req)
        self._finish(req, "abort")
        self.scheduler.retire(req)

    def has_pending(self) -> bool:
        return self.scheduler.has_pending() or self._inflight is not None

    def assert_balanced(self) -> None:
        self.manager.assert_balanced()

    # ------------------------------------------------------------------ the step

    def step(self) -> list[TokenOutput]:
        """Schedules and launches the next step, then returns the tokens of the step before it.

        With ``lookahead`` (the default) the ids a step sampled stay on the device and feed the next
        step directly; the host reads them only after that next step has been launched, so its
        bookkeeping overlaps the GPU's work and outputs arrive one call later.  What follows from
        not knowing the last tokens when scheduling: a request that ends on an eos id has one more
        row in the step already launched (its result is dropped); requests that end by length are
        not scheduled again.  Without lookahead every call returns its own step's tokens."""
        outputs: list[TokenOutput] = []
        t0 = time.perf_counter()
        decision = self.scheduler.schedule()
        launched = None
        try:
            if decision.portions:
                launched = self._launch(decision)
                self.rows_launched += len(decision.portions)
            elif self._inflight is None and self.scheduler.waiting and not self.scheduler.running:
                req = self.scheduler.waiting[0]
                need = self.manager.peak_pages(req.num_tokens, self.scheduler.chunked_budget)
                if any(n > t - self.scheduler.watermark for n, t in zip(need, self.manager.total_pages())):
                    # Not even an empty engine can hold it: it would wait for ever.
                    self.scheduler.waiting.popleft()
                    self._finish(req, "capacity")
                    last = req.generated_ids[-1] if req.generated_ids else -1
                    outputs.append(TokenOutput(req.seq_id, last, True, "capacity"))
            self.host_seconds += time.perf_counter() - t0
            if self.lookahead:
                previous, self._inflight = self._inflight, launched
            else:
                previous = launched
            if previous is not None:
                self._collect(previous, outputs)
        finally:
            for req in [r for r in self.scheduler.running if r.is_finished]:
                self.scheduler.retire(req)
        self.steps += 1
        return outputs

    def _launch(self, decision) -> "_Inflight | None":
        """Feeds the scheduled portions to the step function and launches sampling; nothing is read back."""
        prev = self._inflight
        prev_index = {id(r): i for i, r in enumerate(prev.samplers)} if prev is not None else {}
        entries, samplers = [], []
        for p in decision.portions:
            r = p.request
            from_device = None
            if r.pending and p.start + p.length == r.num_tokens:
                # its newest token is still on the device (sampled by the step in flight)
                if p.length != 1 or id(r) not in prev_index:
                    raise RuntimeError(f"request {r.seq_id}: a token that the host has not read can only be decoded")
                ids, from_device = [0], prev_index[id(r)]
            else:
                ids = r.tokens(p.start, p.length)
            entries.append(StepEntry(r.cache, ids, [p.length - 1] if p.samples else [], from_device))
            if p.samples:
                samplers.append(r)
        logits = self.runner.step(entries, prev.sampled.tokens if prev is not None else None)
        for p in decision.portions:
            p.request.cursor = p.start + p.length
        if not samplers:
            return None
        sampled = self.sampler.launch_async(logits, [r.sampling for r in samplers],
                                            [r.num_generated for r in samplers])
        for r in samplers:
            r.pending += 1
        return _Inflight(samplers, sampled)

    def _collect(self, inflight: "_Inflight", outputs: list[TokenOutput]) -> None:
        """Reads a launched step's sampled ids and records them."""
        for req, tok in zip(inflight.samplers, inflight.sampled.read()):
            req.pending -= 1
            if req.is_finished:
                continue            # it ended on the token before (eos): this row ran for nothing
            self._record(req, tok, outputs)

    def _finish(self, req: Request, reason: str) -> None:
        req.stop_reason = reason
        req.status = RequestStatus.FINISHED

    def _record(self, req: Request, token_id: int, outputs: list[TokenOutput]) -> None:
        req.generated_ids.append(token_id)
        now = time.perf_counter()
        if req.first_token_at is None:
            req.first_token_at = now
        req.last_token_at = now
        if token_id in req.eos_ids:
            self._finish(req, "stop")
        elif len(req.generated_ids) >= req.max_tokens:
            self._finish(req, "length")
        outputs.append(TokenOutput(req.seq_id, token_id, req.is_finished, req.stop_reason))
