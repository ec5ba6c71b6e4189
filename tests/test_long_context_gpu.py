"""A long request (thousands of tokens, hundreds of pages): whole, in large portions with a
decoded tail, against the plain implementation; and a far key that must win over thousands of
others at decode time (a fault in a split, a page or a tile far from the query would lose it)."""

import numpy as np
import pytest

from tests.plain import model as plain
from tests.tiny import TINY_D, make_model_dir, random_tokens, read_weights, sizes_of

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def long_case(tmp_path_factory):
    d = make_model_dir(tmp_path_factory.mktemp("long"), TINY_D)
    w = read_weights(d)
    toks = random_tokens(2500, TINY_D["cfg"].vocab_size, 77)
    ref = plain.forward(sizes_of(TINY_D["cfg"]), w, toks).numpy()
    return d, toks, ref


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 8e-2)])
def test_long_request_cut_in_large_portions_then_decoded(long_case, dtype, tol):
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.replay import TraceSession
    d, toks, ref = long_case
    runner = ModelRunner.from_model_dir(d, dtype=dtype, num_blocks=2560 // 16 + 2, page_size=16, max_requests=2,
                                        max_step_tokens=4096)
    sess = TraceSession(runner)
    cuts = [0, 1000, 1700, 2400]
    steps = [{"step": i, "entries": [{"id": "x", "tokens": toks[a:b], "want": [0, b - a - 1]}], "end": []}
             for i, (a, b) in enumerate(zip(cuts, cuts[1:]))]
    steps += [{"step": 3 + i, "entries": [{"id": "x", "tokens": [toks[2400 + i]], "want": [0]}], "end": []}
              for i in range(100)]
    steps[-1]["end"] = ["x"]
    worst = 0.0
    for s in steps:
        got = sess.step(s)
        e = s["entries"][0]
        start = sum(len(t["entries"][0]["tokens"]) for t in steps[:s["step"]])
        for row, wpos in zip(got, e["want"]):
            worst = max(worst, float(np.abs(row - ref[start + wpos]).max()))
    runner.manager.assert_balanced()
    assert worst < tol, worst
