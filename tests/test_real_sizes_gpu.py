"""Logits at the layer sizes the benchmark runs: Qwen3-8B widths (hidden 4,096, 32 query and 8 kv
heads of 128, feed-forward 12,288, vocabulary 151,936) with 2 of the configuration's 36 layers,
against the plain implementation on the CPU, in float32 and in bfloat16.

The weights are the random-weights mode's: drawn on the device by the engine and, bit for bit the
same, on the host for the plain model, which draws only what it needs (the token table's rows of
the ids in use; the output matrix in slabs).  The shapes are the ones the tiny configurations
cannot reach: the gate/up product as 384 half tiles three to an SM, the down product split over a
cluster at K = 12,288, the output matrix at N = 151,936, TMA decode attention with the splits the
launch plan picks, tcgen05 prefill attention continuing inside a 128-key block, above 32 rows
the library products with the stand-alone norm / rotation / SwiGLU kernels, at 600 rows the gate/up
product alone on the paired tcgen05 kernel, and at 2,100 rows every product of a layer on it with its
fused epilogues.

Tolerances are measured (logits have a standard deviation of 1.3 and reach 6): the float32 engine
differs from the float64 plain result by up to 3.7e-5 (sums over 12,288 terms; relative
root-mean-square 5.5e-6), the bfloat16 engine by up to 7.5e-2 (relative root-mean-square 1.0e-2),
the same whole, in portions and decoding.
"""

import numpy as np
import pytest
import torch

from tests.plain import model as plain
from tests.tiny import random_tokens

pytestmark = pytest.mark.gpu

LAYERS, LAYERS_OF_CONFIG = 2, 36
SEED, SIGMA, SIGMA_NORM = 8, 0.02, 0.1
TOL = {"float32": 1e-4, "bfloat16": 1e-1}
RMS_TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def config():
    from acorninfer_b200.config.model_config import Qwen3Config
    return Qwen3Config(num_hidden_layers=LAYERS, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                       head_dim=128, intermediate_size=12288, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=151936,
                       tie_word_embeddings=False, bos_token_id=None, eos_token_id=())


class PlainSide:
    """The plain model's view of the random model: layer weights held once (in ``dtype``), token-table
    rows drawn on demand, logits through slabs of the output matrix."""

    def __init__(self, dtype):
        from acorninfer_b200.models.decoder import expected_tensors
        from acorninfer_b200.registry import spec_for
        from acorninfer_b200.weights.random_init import random_tensor
        self.cfg = config()
        self.sizes = self.cfg.to_dict()
        self.dtype = dtype
        self.specs = expected_tensors(spec_for(self.cfg))
        self.draw = lambda name, rows=None: random_tensor(name, self.specs[name], SEED, SIGMA, SIGMA_NORM,
                                                          torch.bfloat16, "cpu", rows=rows)
        self.w = {name: self.draw(name).to(dtype) for name in self.specs
                  if name not in ("model.embed_tokens.weight", "lm_head.weight")}
        self.head = self.draw("lm_head.weight")                       # bfloat16, widened slab by slab

    def hidden(self, ids, places):
        """Final normed hidden rows of the sequence ``ids`` at ``places``."""
        rows = {t: self.draw("model.embed_tokens.weight", (t, t + 1))[0] for t in set(ids)}
        embedded = torch.stack([rows[t] for t in ids])
        return plain.final_hidden(self.sizes, self.w, ids, self.dtype, embedded=embedded)[list(places)]

    def head_logits(self, h):
        out = torch.empty(h.shape[0], self.cfg.vocab_size, dtype=self.dtype)
        for r0 in range(0, self.cfg.vocab_size, 16384):
            slab = self.head[r0:r0 + 16384].to(self.dtype)
            out[:, r0:r0 + slab.shape[0]] = h @ slab.T
        return out.double().numpy()

    def logits(self, ids, places):
        return self.head_logits(self.hidden(ids, places))


@pytest.fixture(scope="module")
def plain64():
    return PlainSide(torch.float64)


@pytest.fixture(scope="module")
def plain32():
    return PlainSide(torch.float32)


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def runner(request):
    from acorninfer_b200.engine.runner import ModelRunner
    r = ModelRunner.from_random(config(), SEED, SIGMA, SIGMA_NORM, dtype=request.param, num_blocks=1400, page_size=16,
                                max_requests=64, max_step_tokens=4096)
    yield r
    r.manager.assert_balanced()


def check(got, want, dtype: str, what: str) -> None:
    """The largest difference of any logit, and the root-mean-square difference relative to the logits'
    own (a single wrong key or page moves far more than rounding does)."""
    diff = got.double().cpu().numpy() - want
    w = float(np.abs(diff).max())
    rel = float(np.sqrt((diff ** 2).mean() / (want ** 2).mean()))
    print(f"{what} [{dtype}]: worst |d| = {w:.3e}, rms(d) / rms(logits) = {rel:.3e}")
    assert w < TOL[dtype] and rel < RMS_TOL[dtype], f"{what}: worst |d| = {w:.3e}, relative rms = {rel:.3e}"


def dtype_of(runner) -> str:
    return "float32" if runner.dtype == torch.float32 else "bfloat16"


def test_sizes_are_the_benchmarks():
    """The configuration named here is the benchmark's but for the number of layers."""
    import bench
    cfg = config().to_dict()
    for key, value in bench.QWEN3_8B.items():
        if key not in ("num_hidden_layers", "bos_token_id", "eos_token_id"):
            assert cfg[key] == value, key
    assert bench.QWEN3_8B["num_hidden_layers"] == LAYERS_OF_CONFIG


def test_a_prompt_whole_and_in_portions(runner, plain64):
    """300 tokens in one step; and as 200 + 60 + 40, where the second and third portions start inside
    the request and inside a block of 128 keys (tcgen05 attention with an offset)."""
    from acorninfer_b200.engine.batch import StepEntry
    ids = random_tokens(300, runner.vocab_size, 41)
    places = [0, 1, 127, 128, 199, 200, 259, 260, 299]
    want = plain64.logits(ids, places)
    rc = runner.open("whole")
    got = runner.step([StepEntry(rc, ids, places)])
    runner.close(rc)
    check(got, want, dtype_of(runner), "whole")
    rc = runner.open("portions")
    parts, at = [], 0
    for n in (200, 60, 40):
        mine = [p - at for p in places if at <= p < at + n]
        parts.append(runner.step([StepEntry(rc, ids[at:at + n], mine)]))
        at += n
    runner.close(rc)
    check(torch.cat(parts), want, dtype_of(runner), "portions 200 + 60 + 40")


_LONG = {}


def test_a_long_prompt_on_the_paired_kernel(runner, plain64):
    """2,100 tokens in one step: in bfloat16 every product of the layers runs on the paired tcgen05 kernel
    (nine token tiles: the last one holds 52 tokens) with q/k norm, rotation and the cache write, SwiGLU
    and the residual sums with the next norm's sums as its epilogues; in float32 on the tiled CUDA-core
    product.  Places at the edges of the 256-token tiles and of the 128-key attention blocks."""
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.kernels import ops
    ids = random_tokens(2100, runner.vocab_size, 43)
    places = [0, 1, 127, 128, 255, 256, 1023, 1024, 2047, 2048, 2099]
    if "want" not in _LONG:
        _LONG["want"] = plain64.logits(ids, places)
    before = dict(ops.COUNTS)
    rc = runner.open("long")
    got = runner.step([StepEntry(rc, ids, places)])
    runner.close(rc)
    ran = {k: v - before.get(k, 0) for k, v in ops.COUNTS.items() if v - before.get(k, 0)}
    if runner.dtype == torch.bfloat16:
        # the last layer's down product has no norm after it for all rows (the final norm takes the wanted
        # rows only): it adds to the residual stream through the library product's C operand
        assert ran.get("gemm_tc_pair") == 3 * LAYERS - 1 and ran.get("gemm_tc_pair_qkv_rope") == LAYERS
        assert "swiglu" not in ran and "qk_rope_kv" not in ran
        ops.raise_on_kernel_error()
    check(got, _LONG["want"], dtype_of(runner), "2,100 tokens whole")


def test_a_prompt_of_600_tokens_with_gate_up_alone_on_the_paired_kernel(runner, plain64):
    """600 tokens in one step: too few for every product of a layer to fill the device, enough for the
    gate/up product, which in bfloat16 runs on the paired kernel with SwiGLU while the others stay on the
    library (three token tiles, the last one holding 88 tokens)."""
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.kernels import ops
    ids = random_tokens(600, runner.vocab_size, 47)
    places = [0, 255, 256, 511, 512, 599]
    want = plain64.logits(ids, places)
    before = dict(ops.COUNTS)
    rc = runner.open("mid")
    got = runner.step([StepEntry(rc, ids, places)])
    runner.close(rc)
    ran = {k: v - before.get(k, 0) for k, v in ops.COUNTS.items() if v - before.get(k, 0)}
    if runner.dtype == torch.bfloat16:
        assert ran.get("gemm_tc_pair") == LAYERS and "gemm_tc_pair_qkv_rope" not in ran and "swiglu" not in ran
        assert ran.get("qk_rope_kv") == LAYERS
        ops.raise_on_kernel_error()
    check(got, want, dtype_of(runner), "600 tokens whole")
    # alone in its step, the prompt was padded to 640 tokens; the same shape again is captured, then replayed
    # (the paired kernel inside a CUDA graph), and the padding's keys and values stay out of every result
    replays = runner.graph_replays
    for again in ("captured", "replayed"):
        rc = runner.open("mid " + again)
        got = runner.step([StepEntry(rc, ids, places)]).clone()
        nxt = runner.step([StepEntry(rc, [ids[0]], [0])]).clone()      # a decoded token lands in a slot the padding wrote
        runner.close(rc)
        check(got, want, dtype_of(runner), "600 tokens, " + again)
        if again == "captured":
            want_next = plain64.logits(ids + [ids[0]], [600])
        check(nxt, want_next, dtype_of(runner), "the token after, " + again)
    assert runner.graph_replays >= replays + 1
    ops.raise_on_kernel_error()


def decode_case(runner, side, rows, prompt_lens, steps, seed):
    """``rows`` requests: prompts in steps of up to eight requests, then ``steps`` decode steps of all of
    them together; the logits of every decoded token against the plain model."""
    from acorninfer_b200.engine.batch import StepEntry
    seqs = [random_tokens(prompt_lens[i % len(prompt_lens)] + steps, runner.vocab_size, seed + i) for i in range(rows)]
    rcs = [runner.open(f"d{rows}_{i}") for i in range(rows)]
    for i in range(0, rows, 8):
        runner.step([StepEntry(rcs[j], seqs[j][:len(seqs[j]) - steps], []) for j in range(i, min(rows, i + 8))])
    got = []
    for k in range(steps):
        got.append(runner.step([StepEntry(rc, [s[len(s) - steps + k]], [0]) for rc, s in zip(rcs, seqs)]).clone())
    for rc in rcs:
        runner.close(rc)
    want = side.head_logits(torch.cat([side.hidden(s, range(len(s) - steps, len(s))) for s in seqs]))
    mine = torch.stack([got[k][j] for j in range(rows) for k in range(steps)])
    check(mine, want, dtype_of(runner), f"{rows} requests decoding")


def test_eight_requests_decoding(runner, plain64):
    """The benchmark's batch: the fused tcgen05 path (q/k/v with norm, rotation and cache write; o with
    the residual sum and norm; gate/up with SwiGLU as half tiles; down split over a cluster at
    K = 12,288; the output matrix at N = 151,936), TMA decode attention in several splits, captured."""
    from acorninfer_b200.kernels.ops import gemm_tc_plan
    assert gemm_tc_plan(8, 24576, 4096) == (2, 3) and gemm_tc_plan(8, 4096, 12288)[0] >= 2
    replays = runner.graph_replays
    decode_case(runner, plain64, 8, (300, 41, 130, 257, 64, 199, 17, 90), 5, 500)
    assert runner.graph_replays >= replays + 3


@pytest.mark.parametrize("rows", [40, 64])
def test_many_requests_decoding(runner, plain32, rows):
    """Above 32 rows: library products with the residual as C operand, the stand-alone kernels, the
    buckets of 40 and 64 rows, the decode kernel's splits for that many rows."""
    if runner.dtype == torch.float32:
        pytest.skip("the float32 engine has one path for every row count; it is checked at 8 rows")
    decode_case(runner, plain32, rows, (21, 33, 18, 40, 27), 3, 7000 + rows)
