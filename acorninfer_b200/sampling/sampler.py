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


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], counters: list[int],
               want_logprobs: bool = False) -> tuple[list[int], list[float] | None]:
        """``logits`` float32 [R, vocab]; one SamplingParams and one draw counter per row."""
        R = logits.shape[0]
        if len(params) != R or len(counters) != R:
            raise ValueError("one SamplingParams and one counter per logits row")
        host = torch.empty((5, R), dtype=torch.float64)
        for i, (p, c) in enumerate(zip(params, counters)):
            host[0, i], host[1, i], host[2, i] = p.temperature, p.top_k, p.top_p
        dev = host.to(self.device, non_blocking=False)
        seeds = torch.tensor([p.seed & (2 ** 63 - 1) for p in params], dtype=torch.int64).to(self.device)
        ctrs = torch.tensor([int(c) for c in counters], dtype=torch.int64).to(self.device)
        tokens, logprobs = ops.sample(logits, dev[0].float().contiguous(), dev[1].to(torch.int32).contiguous(),
                                      dev[2].float().contiguous(), seeds, ctrs, want_logprobs)
        toks = tokens.tolist()
        if any(t < 0 for t in toks):
            raise ValueError("logits contain NaN or infinity: the model's forward pass is broken")
        return toks, (logprobs.tolist() if want_logprobs else None)

    def greedy(self, logits: torch.Tensor) -> list[int]:
        R = logits.shape[0]
        return self.sample(logits, [SamplingParams(temperature=0.0)] * R, [0] * R)[0]
