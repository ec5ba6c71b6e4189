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


def run_cut(tiny, model_dir, steps, dtype, max_requests=4, watch=None):
    """Replays ``steps`` on a pool just large enough for the trace.  ``watch(session, msg)`` is called
    after every step, before the step's ended requests are closed."""
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.replay import TraceSession

    pool_tokens = traces.max_live_tokens(steps)
    runner = ModelRunner.from_model_dir(model_dir, dtype=dtype, num_blocks=-(-pool_tokens // tiny["page_size"]),
                                        page_size=tiny["page_size"], max_requests=max_requests, max_step_tokens=4096)
    session = TraceSession(runner)

    def step(msg):
        if watch is None:
            return session.step(msg)
        out = session.step(dict(msg, end=[]))
        watch(session, msg)
        session.step({"entries": [], "end": msg["end"]})
        return out

    got = traces.collect(step, steps)
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
    """In the mixed trace physical pages really serve several requests one after another: seen on the
    cache manager's block tables while the trace runs, whatever order the pool hands pages out in."""
    tiny, d, reqs, _ = tiny_case
    steps = traces.mixed(reqs)
    assert traces.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for t in reqs.values())
    served: dict[int, set] = {}

    def watch(session, msg):
        for rid, rc in session.live.items():
            for page in rc.tables[0]:
                served.setdefault(page, set()).add(rid)

    run_cut(tiny, d, steps, "float32", watch=watch)
    assert sum(1 for users in served.values() if len(users) >= 2) >= 2, served


# ------------------------------------------------------------------ schedules of a serving engine, head size 128


@pytest.fixture(scope="module")
def tiny_d_long(tmp_path_factory):
    """Tiny D (head size 128: the tcgen05 prefill and TMA decode kernels) with requests long enough
    for portions of 32 to 60 tokens that start inside a request and inside a 128-key block."""
    tiny = TINIES["tiny_d"]
    d = make_model_dir(tmp_path_factory.mktemp("tiny_d_long"), tiny)
    w = read_weights(d)
    reqs = {f"q{i}": random_tokens(n, tiny["cfg"].vocab_size, 2000 + i) for i, n in enumerate([230, 171, 140, 260, 97, 205])}
    ref = {rid: plain.forward(sizes_of(tiny["cfg"]), w, toks).numpy() for rid, toks in reqs.items()}
    return tiny, d, reqs, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_beside_decoded_tokens(tiny_d_long, dtype):
    """What a serving engine does at every step of a chunked prefill: portions of up to 60 tokens of
    some requests (on the tcgen05 kernel from 32 tokens on, starting anywhere) in one step, and one
    output tensor, with single decoded tokens of others (TMA decode kernel)."""
    from acorninfer_b200.kernels import ops
    tiny, d, reqs, ref = tiny_d_long
    steps = traces.mixed(reqs, seed=3, prompt_frac=0.7, min_portion=20, max_portion=60, stagger=5)
    both = [s for s in steps if any(len(e["tokens"]) >= 32 for e in s["entries"])
            and any(len(e["tokens"]) == 1 for e in s["entries"])]
    assert len(both) >= 5                                     # the trace has the steps this test is about
    before = dict(ops.COUNTS)
    got = run_cut(tiny, d, steps, dtype)
    ran = {k: v - before.get(k, 0) for k, v in ops.COUNTS.items()}
    if dtype == "bfloat16":
        assert ran.get("attention_prefill_tc", 0) >= 10 and ran.get("attention_decode_tma", 0) >= 10
        assert ran.get("attention_plain", 0) == 0
    assert len(got) == sum(len(t) for t in reqs.values())
    for (rid, pos), row in got.items():
        diff = np.abs(row - ref[rid][pos]).max()
        assert diff < TOL[dtype], f"{dtype}: request {rid} position {pos}: |d|={diff:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_forty_requests_decoding(tmp_path_factory, dtype):
    """A decode batch above 32 rows: the padded bucket of 40 (and 48 when 41 are live), its padding
    rows, the library products with the residual as their C operand, the stand-alone norm / rotation /
    SwiGLU kernels at decode shape and captured graphs, all against the plain model."""
    tiny = TINIES["tiny_d"]
    d = make_model_dir(tmp_path_factory.mktemp("forty"), tiny)
    w = read_weights(d)
    V = tiny["cfg"].vocab_size
    reqs = {f"m{i}": random_tokens(14 + (5 * i) % 23, V, 3000 + i) for i in range(41)}
    ref = {rid: plain.forward(sizes_of(tiny["cfg"]), w, toks).numpy() for rid, toks in reqs.items()}
    steps, at = [], {rid: 0 for rid in reqs}
    # prompts: all but the last 8 tokens of each request, five requests a step
    rids = list(reqs)
    for i in range(0, len(rids), 5):
        entries = []
        for rid in rids[i:i + 5]:
            n = len(reqs[rid]) - 8
            entries.append({"id": rid, "tokens": reqs[rid][:n], "want": [n - 1]})
            at[rid] = n
        steps.append({"entries": entries, "end": []})
    # then every live request decodes: 41 rows (bucket 48) for one step, 40 rows (bucket 40) afterwards
    for k in range(8):
        live = rids if k == 0 else rids[:40]
        entries = [{"id": rid, "tokens": [reqs[rid][at[rid]]], "want": [0]} for rid in live]
        for rid in live:
            at[rid] += 1
        steps.append({"entries": entries, "end": [rids[40]] if k == 0 else []})
    steps[-1]["end"] = rids[:40]
    for i, s in enumerate(steps):
        s["step"] = i
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.replay import TraceSession
    runner = ModelRunner.from_model_dir(d, dtype=dtype, num_blocks=41 * 3 + 2, page_size=16, max_requests=41)
    got = traces.collect(TraceSession(runner).step, steps)
    runner.manager.assert_balanced()
    assert runner.graph_replays >= 5                           # the bucket of 40 was captured and replayed
    assert len(got) == 41 + 41 + 7 * 40
    for (rid, pos), row in got.items():
        diff = np.abs(row - ref[rid][pos]).max()
        assert diff < TOL[dtype], f"{dtype}: request {rid} position {pos}: |d|={diff:.3e}"


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


@pytest.mark.parametrize("which", ["tiny_d", "tiny_c"])
@pytest.mark.parametrize("cut", ["whole", "mixed_long"])
def test_paired_kernel_path_matches_plain(monkeypatch, tmp_path, cut, which):
    """Steps of more than 32 rows on the paired tcgen05 kernel with its fused epilogues (which the engine
    takes by itself only where its tiles fill the device: thousands of rows at real widths): forced here
    for every such step of the head-size-128 configuration, whole prompts and long portions beside
    decoded tokens, against the plain model.  The configuration with head size 48 and a feed-forward
    width that is no multiple of 64 takes the kernel's plain form fed with un-normalised rows, followed
    by the stand-alone rotation and SwiGLU kernels."""
    from acorninfer_b200.kernels import ops
    monkeypatch.setattr(ops, "GEMM_PAIR_MIN_ROWS", 33)
    monkeypatch.setattr(ops, "GEMM_PAIR_MIN_FILL", 0.0)
    monkeypatch.setattr(ops, "GEMM_PAIR_MIN_FILL_ALONE", 0.0)
    monkeypatch.setattr(ops, "GEMM_PAIR_ALONE_MIN_K", 0)
    tiny = TINIES[which]
    d = make_model_dir(tmp_path, tiny)
    w = read_weights(d)
    lengths = [40, 157, 70, 33, 300, 64]
    reqs = {f"r{i}": random_tokens(n, tiny["cfg"].vocab_size, 2000 + i) for i, n in enumerate(lengths)}
    ref = {rid: plain.forward(sizes_of(tiny["cfg"]), w, toks).numpy() for rid, toks in reqs.items()}
    steps = traces.whole(reqs) if cut == "whole" else traces.mixed(reqs, max_portion=60, min_portion=34, stagger=2)
    before = dict(ops.COUNTS)
    got = run_cut(tiny, d, steps, "bfloat16")
    ran = {k: v - before.get(k, 0) for k, v in ops.COUNTS.items()}
    assert ran.get("gemm_tc_pair", 0) > 0
    if which == "tiny_d":
        assert ran.get("gemm_tc_pair_qkv_rope", 0) > 0 and ran.get("rope_table", 0) > 0 and not ran.get("swiglu", 0)
    else:
        assert ran.get("qk_rope_kv", 0) > 0 and ran.get("swiglu", 0) > 0 and not ran.get("gemm_tc_pair_qkv_rope", 0)
    assert len(got) == sum(lengths)
    for (rid, pos), row in got.items():
        diff = np.abs(row - ref[rid][pos]).max()
        assert diff < TOL["bfloat16"], f"{cut}: request {rid} position {pos}: |d|={diff:.3e}"
