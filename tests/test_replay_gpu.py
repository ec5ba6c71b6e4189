"""Replay on the GPU against the plain implementation: the same requests whole, with the
last 32 tokens one by one, in portions of changing size, and mixed with other requests in a
pool so small that pages are used again; in float32 and in bfloat16; on three tiny
configurations that differ in every size and option.

Tolerances are measured, not guessed (logit magnitudes are about 2):
float32 differs from the float64 plain result by 4e-7 .. 1.6e-6 (summation order);
bfloat16 by 3e-3 .. 1.5e-2 (bfloat16 activations between the matrix products).
Between two cuts of the same requests the engine's float32 results agree to 1e-5.
"""

import numpy as np
import pytest
import torch

from tests import traces
from tests.plain import model as plain
from tests.tiny import TINIES, make_model_dir, random_tokens, read_weights, sizes_of

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 6e-2}
LENGTHS = [40, 57, 70, 33, 90, 64]


@pytest.fixture(scope="module", params=list(TINIES))
def tiny_case(request, tmp_path_factory):
    tiny = TINIES[request.param]
    d = make_model_dir(tmp_path_factory.mktemp(request.param), tiny)
    w = read_weights(d)
    reqs = {f"r{i}": random_tokens(n, tiny["cfg"].vocab_size, 1000 + i) for i, n in enumerate(LENGTHS)}
    ref = {rid: plain.forward(sizes_of(tiny["cfg"]), w, toks).numpy() for rid, toks in reqs.items()}
    return tiny, d, reqs, ref


def run_cut(tiny, model_dir, steps, dtype):
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.replay import TraceSession

    pool_tokens = traces.max_live_tokens(steps)
    runner = ModelRunner.from_model_dir(model_dir, dtype=dtype, num_blocks=-(-pool_tokens // tiny["page_size"]),
                                        page_size=tiny["page_size"], max_requests=4, max_step_tokens=4096)
    got = traces.collect(TraceSession(runner).step, steps)
    runner.manager.assert_balanced()
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["whole", "decode_tail", "portions", "mixed"])
def test_cut_matches_plain(tiny_case, cut, dtype):
    tiny, d, reqs, ref = tiny_case
    steps = getattr(traces, cut)(reqs)
    got = run_cut(tiny, d, steps, dtype)
    assert len(got) == sum(len(t) for t in reqs.values())
    for (rid, pos), row in got.items():
        diff = np.abs(row - ref[rid][pos]).max()
        assert diff < TOL[dtype], f"{cut} {dtype}: request {rid} position {pos}: |d|={diff:.3e}"


def test_cuts_agree_with_each_other_float32(tiny_case):
    tiny, d, reqs, _ = tiny_case
    base = run_cut(tiny, d, traces.whole(reqs), "float32")
    for cut in ("decode_tail", "portions", "mixed"):
        other = run_cut(tiny, d, getattr(traces, cut)(reqs), "float32")
        for key, row in base.items():
            assert np.abs(row - other[key]).max() < 1e-5, f"{cut}: {key}"


def test_mixed_trace_reuses_pages(tiny_case):
    """The mixed trace's pool is smaller than the sum of all requests, so later requests
    can only run on pages that earlier ones gave back."""
    tiny, _, reqs, _ = tiny_case
    steps = traces.mixed(reqs)
    assert traces.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for t in reqs.values())


def test_weights_stored_in_float32_stay_float32_under_a_bfloat16_engine(tmp_path):
    """A folder whose tensors are stored in 32 bits: the bfloat16 engine keeps them so and multiplies
    those matrices in float32 (activations between the parts are still bfloat16)."""
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.replay import TraceSession
    from acorninfer_b200.weights.random_init import write_random_model
    from tests.tiny import TINY_A

    tiny = TINY_A
    d = write_random_model(tmp_path / "m32", tiny["cfg"], tiny["seed"], tiny["sigma"], tiny["sigma_norm"], torch.float32)
    w = read_weights(d)
    assert all(t.dtype == torch.float32 for t in w.values())
    reqs = {"a": random_tokens(45, tiny["cfg"].vocab_size, 1), "b": random_tokens(38, tiny["cfg"].vocab_size, 2)}
    ref = {rid: plain.forward(sizes_of(tiny["cfg"]), w, toks).numpy() for rid, toks in reqs.items()}
    steps = traces.decode_tail(reqs)
    runner = ModelRunner.from_model_dir(d, dtype="bfloat16", num_blocks=-(-traces.max_live_tokens(steps) // 4),
                                        page_size=4, max_requests=2)
    assert runner.decoder.embedding.dtype == torch.float32 and runner.decoder.blocks[0].mixer.w_qkv.dtype == torch.float32
    got = traces.collect(TraceSession(runner).step, steps)
    for (rid, pos), row in got.items():
        assert np.abs(row - ref[rid][pos]).max() < 2e-2, (rid, pos)
