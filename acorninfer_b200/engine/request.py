"""A request inside the engine: its tokens, its sampling parameters, where it stands.

Reference: ``Sequence`` / ``RequestStatus`` in ``acorninfer/engine/sequence.py:12-46``.  The
three status values and the fields ``seq_id .. last_token_at`` with ``num_tokens``, ``all_ids`` and
``is_finished`` are the reference's interface, kept name for name because its callers (the
benchmark protocol's ``engine.seqs[i]``, the time stamps) read them; ``cursor``, ``pending``,
``exhausted``, ``tokens()``, ``preemptions`` and ``cache`` are this engine's.
``cursor`` counts the tokens of ``all_ids`` whose keys and values are in the cache; a
request whose pages were taken away (preemption) starts again from cursor 0 over
``all_ids`` (prompt plus what it has generated), which recomputes the same cache.
"""

from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field

from ..sampling.params import SamplingParams


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass(eq=False)          # requests are compared by identity (field-wise equality would walk the token lists)
class Request:
    seq_id: int
    prompt_ids: list[int]
    sampling: SamplingParams
    max_tokens: int
    eos_ids: frozenset[int]
    generated_ids: list[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    stop_reason: str | None = None
    cursor: int = 0                      # tokens of all_ids already in the cache
    pending: int = 0                     # tokens sampled on the device that the host has not read yet (0 or 1)
    cache: object = None                 # RequestCache while running
    preemptions: int = 0
    created_at: float = field(default_factory=time.perf_counter)
    first_token_at: float | None = None
    last_token_at: float | None = None

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.generated_ids) + self.pending

    @property
    def num_generated(self) -> int:
        return len(self.generated_ids) + self.pending

    @property
    def exhausted(self) -> bool:
        """All tokens it may generate are sampled; the last one may still be on its way to the host."""
        return self.num_generated >= self.max_tokens

    @property
    def all_ids(self) -> list[int]:
        return self.prompt_ids + self.generated_ids

    def tokens(self, start: int, length: int) -> list[int]:
        """``all_ids[start:start + length]`` without building the whole list."""
        n_prompt = len(self.prompt_ids)
        end = start + length
        if end <= n_prompt:
            return self.prompt_ids[start:end]
        if start >= n_prompt:
            return self.generated_ids[start - n_prompt:end - n_prompt]
        return self.prompt_ids[start:] + self.generated_ids[:end - n_prompt]

    @property
    def is_finished(self) -> bool:
        return self.status is RequestStatus.FINISHED
