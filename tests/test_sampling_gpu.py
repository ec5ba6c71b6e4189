"""The sampling kernel against the plain processing (temperature, top-k, top-p) with the
same uniform numbers, and its greedy, tie and bad-input behaviour."""

import pytest
import torch

from tests.plain import model as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run(logits, temperature, top_k, top_p, seeds, counters, logprobs=False):
    from acorninfer_b200.kernels import ops
    R = logits.shape[0]
    f = lambda v, dt: torch.tensor(v if isinstance(v, list) else [v] * R, dtype=dt, device=DEV)
    toks, lps = ops.sample(logits.to(DEV), f(temperature, torch.float32), f(top_k, torch.int32),
                           f(top_p, torch.float32), f(seeds, torch.int64), f(counters, torch.int64), logprobs)
    return toks.tolist(), (lps.tolist() if logprobs else None)


def test_greedy_takes_the_first_of_equal_maxima():
    x = torch.randn(5, 1003)
    x[0, 77] = x[0, 900] = 9.0
    x[3, 0] = 9.0
    toks, _ = run(x, 0.0, 0, 1.0, 0, 0)
    assert toks == [77] + x[1:].argmax(-1).tolist()


def test_bad_logits_are_flagged_not_sampled():
    x = torch.randn(3, 50)
    x[1, 4] = float("nan")
    x[2, 9] = float("inf")
    toks, _ = run(x, 1.0, 0, 1.0, 0, 0)
    assert toks[0] >= 0 and toks[1] == -1 and toks[2] == -1


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.7, 0, 1.0), (1.0, 5, 1.0), (1.3, 0, 0.8), (0.9, 40, 0.6),
                                                     (0.5, 1, 1.0), (1.0, 0, 0.05)])
def test_sampling_matches_plain_with_the_same_uniforms(temperature, top_k, top_p):
    from acorninfer_b200.kernels import ops
    torch.manual_seed(5)
    R, V = 24, 1531
    x = 3 * torch.randn(R, V)
    seeds = list(range(100, 100 + R))
    counters = list(range(R))
    toks, lps = run(x, temperature, top_k, top_p, seeds, counters, logprobs=True)
    checked = 0
    for r in range(R):
        processed = plain.process_logits(x[r], temperature, top_k, top_p)
        u = ops.uniform(seeds[r], counters[r])
        assert 0.0 <= u < 1.0
        want, want_lp, margin = plain.sample_with_uniform(processed, u)
        assert torch.isfinite(processed[toks[r]]), "the kernel chose a token that top-k/top-p removed"
        if margin > 1e-4:                       # away from a CDF step the choice is unambiguous
            assert toks[r] == want
            assert abs(lps[r] - want_lp) < 1e-3
            checked += 1
    assert checked >= R // 2


def test_draws_follow_the_distribution_and_do_not_depend_on_the_batch():
    V = 7
    x = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5, 1.5, -3.0]]).repeat(4000, 1)
    toks, _ = run(x, 1.0, 0, 1.0, 11, list(range(4000)))
    freq = torch.bincount(torch.tensor(toks), minlength=V).double() / 4000
    assert (freq - x[0].double().softmax(-1)).abs().max() < 0.03
    alone, _ = run(x[:1], 1.0, 0, 1.0, 11, [123])
    assert alone[0] == toks[123]
