"""Per-request sampling parameters.

Names and defaults as in the reference's ``SamplingParams`` (``acorninfer/sampler.py:18-22``):
``temperature`` (0 selects greedy, as the reference's callers decide in
``acorninfer/engine/executor.py:128-138``), ``top_p`` in (0, 1], ``top_k`` (0 disables).
``seed`` is added: every request draws from its own counter-based stream, so its tokens
do not depend on what else is in the batch.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int = 0

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0 (0 = greedy)")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0 (0 disables)")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0
