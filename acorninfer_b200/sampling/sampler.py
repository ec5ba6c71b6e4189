"""Token choice for the rows of a step, on the device.

One kernel launch chooses a token for every row: argmax for greedy rows, otherwise
temperature -> top-k -> top-p -> softmax -> draw, in the reference's order
(``acorninfer/sampler.py:38-67``).  The draw uses a uniform number that is a function of
(request seed, number of tokens the request has drawn so far): the reference draws from
torch's global generator (``acorninfer/engine/executor.py:132-135``), which makes a
request's tokens depend on its neighbours; here they do not.  The result comes back in one
device-to-host copy per step.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .params import SamplingParams


class Sampled:
    """Ids a step sampled: on the device (``tokens``), and on their way to a pinned host buffer; the
    copy was queued right behind the sampling kernel, so it does not wait for later steps."""

    def __init__(self, tokens: torch.Tensor, host: torch.Tensor, event: torch.cuda.Event):
        self.tokens, self.host, self.event = tokens, host, event

    def read(self) -> list[int]:
        self.event.synchronize()
        ops.raise_on_kernel_error()
        toks = self.host.tolist()
        if any(t < 0 for t in toks):
            raise ValueError("logits contain NaN or infinity: the model's forward pass is broken")
        return toks


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._greedy: dict[int, tuple] = {}      # rows -> constant parameter tensors of an all-greedy step
        self._pinned: list[torch.Tensor] = []    # ring of pinned host buffers for the sampled ids
        self._next = 0

    def _host_buffer(self, rows: int) -> torch.Tensor:
        if not self._pinned or self._pinned[0].numel() < rows:
            size = max(256, 1 << (rows - 1).bit_length())
            self._pinned = [torch.empty(size, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._next = (self._next + 1) % len(self._pinned)
        return self._pinned[self._next][:rows]

    def launch_async(self, logits: torch.Tensor, params: list[SamplingParams], counters: list[int]) -> Sampled:
        """Samples on the device and queues the copy of the ids to the host; ``Sampled.read`` waits for
        that copy only."""
        tokens, _ = self.launch(logits, params, counters)
        host = self._host_buffer(tokens.numel())
        host.copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return Sampled(tokens, host, event)

    def _greedy_params(self, R: int):
        got = self._greedy.get(R)
        if got is None:
            z = lambda dt: torch.zeros(R, dtype=dt, device=self.device)
            got = (z(torch.float32), z(torch.int32), torch.ones(R, dtype=torch.float32, device=self.device),
                   z(torch.int64), z(torch.int64))
            self._greedy[R] = got
        return got

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], counters: list[int],
               want_logprobs: bool = False) -> tuple[list[int], list[float] | None]:
        """``logits`` float32 [R, vocab]; one SamplingParams and one draw counter per row."""
        tokens, logprobs = self.launch(logits, params, counters, want_logprobs)
        return self.read(tokens), (logprobs.tolist() if want_logprobs else None)

    @staticmethod
    def read(tokens: torch.Tensor) -> list[int]:
        """Brings sampled ids to the host (waits for the step that sampled them)."""
        toks = tokens.tolist()
        ops.raise_on_kernel_error()
        if any(t < 0 for t in toks):
            raise ValueError("logits contain NaN or infinity: the model's forward pass is broken")
        return toks

    def launch(self, logits: torch.Tensor, params: list[SamplingParams], counters: list[int],
               want_logprobs: bool = False) -> tuple[torch.Tensor, torch.Tensor | None]:
        """Launches the sampling kernel and returns the ids (int32, on the device) without waiting."""
        R = logits.shape[0]
        if len(params) != R or len(counters) != R:
            raise ValueError("one SamplingParams and one counter per logits row")
        if all(p.greedy for p in params):
            temperature, top_k, top_p, seeds, ctrs = self._greedy_params(R)
        else:
            dev = self.device
            temperature = torch.tensor([p.temperature for p in params], dtype=torch.float32).to(dev, non_blocking=True)
            top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32).to(dev, non_blocking=True)
            top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32).to(dev, non_blocking=True)
            seeds = torch.tensor([p.seed & (2 ** 63 - 1) for p in params], dtype=torch.int64).to(dev, non_blocking=True)
            ctrs = torch.tensor([int(c) for c in counters], dtype=torch.int64).to(dev, non_blocking=True)
        return ops.sample(logits, temperature, top_k, top_p, seeds, ctrs, want_logprobs)
