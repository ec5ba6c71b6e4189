"""Which kernel a path really takes: a test that passes on a slower stand-in proves nothing about
the kernel it was written for.  The counters in ``kernels.ops.COUNTS`` are read around small runs."""

import pytest
import torch

from tests.tiny import TINY_B, TINY_D, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu


def counts_of(fn):
    from acorninfer_b200.kernels import ops
    before = dict(ops.COUNTS)
    fn()
    return {k: v - before.get(k, 0) for k, v in ops.COUNTS.items() if v - before.get(k, 0)}


def runner_for(tmp_path, tiny, dtype, **kw):
    from acorninfer_b200.engine.runner import ModelRunner
    d = make_model_dir(tmp_path / f"m_{dtype}", tiny)
    return ModelRunner.from_model_dir(d, dtype=dtype, num_blocks=64, page_size=tiny["page_size"], max_requests=4, **kw)


def test_head_size_128_takes_the_tcgen05_and_tma_kernels(tmp_path):
    from acorninfer_b200.engine.batch import StepEntry
    tiny = TINY_D
    V = tiny["cfg"].vocab_size
    runner = runner_for(tmp_path, tiny, "bfloat16", decode_graph=False)
    a, b = runner.open("a"), runner.open("b")
    layers = tiny["cfg"].num_hidden_layers
    # a prompt of 40 tokens beside one of 5: long rows on the tcgen05 kernel, short ones on mma.sync
    c = counts_of(lambda: runner.step([StepEntry(a, random_tokens(40, V, 1), [39]), StepEntry(b, random_tokens(5, V, 2), [4])]))
    assert c.get("attention_prefill_tc") == layers and c.get("attention_prefill") == layers
    assert "attention_plain" not in c and "attention_decode" not in c
    assert c.get("gemm_tc") == 1                    # 45 rows: the library product; only the two wanted rows' logits
    # two decoded tokens: TMA decode kernel, tcgen05 products with fused epilogues, no norm kernel between layers
    c = counts_of(lambda: runner.step([StepEntry(a, [3], [0]), StepEntry(b, [4], [0])]))
    assert c.get("attention_decode_tma") == layers and "attention_prefill_tc" not in c and "attention_plain" not in c
    assert c.get("gemm_tc") == 3 * layers + 1       # o, gate_up(+SwiGLU), down per layer, and the output matrix
    assert c.get("gemm_tc_qkv_rope") == layers      # q/k-norm, rotation and the cache write ride on the qkv product
    assert "swiglu" not in c and "qk_rope_kv" not in c and c.get("add_rmsnorm") == 2      # first norm and final norm only
    # a mixed step: the decoded token through the decode kernel, the portion through a prefill kernel
    c = counts_of(lambda: runner.step([StepEntry(a, [5], [0]), StepEntry(b, random_tokens(33, V, 3), [])]))
    assert c.get("attention_decode_tma") == layers and c.get("attention_prefill_tc") == layers


def test_float32_takes_only_the_true_32_bit_kernels(tmp_path):
    from acorninfer_b200.engine.batch import StepEntry
    tiny = TINY_B
    runner = runner_for(tmp_path, tiny, "float32")
    a = runner.open("a")
    before_mm = torch.backends.cuda.matmul.allow_tf32
    c = counts_of(lambda: (runner.step([StepEntry(a, random_tokens(20, tiny["cfg"].vocab_size, 1), [19])]),
                           runner.step([StepEntry(a, [7], [0])])))
    layers = tiny["cfg"].num_hidden_layers
    assert c.get("gemm_f32") == 2 * (4 * layers + 1) and c.get("attention_plain") == 2 * layers
    assert not any(k.startswith(("gemm_tc", "attention_decode", "attention_prefill")) for k in c)
    assert torch.backends.cuda.matmul.allow_tf32 == before_mm


def test_other_head_sizes_take_the_cp_async_decode_kernel_and_captured_steps_are_replayed(tmp_path):
    from acorninfer_b200.engine.batch import StepEntry
    tiny = TINY_B                                    # head size 32
    runner = runner_for(tmp_path, tiny, "bfloat16")
    a = runner.open("a")
    runner.step([StepEntry(a, random_tokens(9, tiny["cfg"].vocab_size, 1), [])])
    c = counts_of(lambda: [runner.step([StepEntry(a, [t], [0])]) for t in (1, 2, 3, 4, 5)])
    assert runner.graph_replays == 3                 # seen, captured, then replayed three times
    assert c.get("attention_decode", 0) >= 2 * tiny["cfg"].num_hidden_layers and "attention_decode_tma" not in c


def test_a_kernel_that_gives_up_a_wait_becomes_an_exception_at_the_next_read(tmp_path):
    """Kernels report a bounded wait that gave up through a word of pinned host memory.  A kernel
    that only reports (nothing goes wrong on the device) shows the way from there to the host."""
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.kernels import ops
    from acorninfer_b200.sampling.sampler import Sampler
    ops.raise_on_kernel_error()                          # nothing reported so far
    ops.error_word_selftest(7)
    torch.cuda.synchronize()
    with pytest.raises(ops.KernelError, match="self-test.*point 7"):
        ops.raise_on_kernel_error()
    ops.raise_on_kernel_error()                          # reading clears it
    # the sampler's read is such a point
    ops.error_word_selftest(3)
    ids = torch.zeros(2, dtype=torch.int32, device="cuda:0")
    with pytest.raises(ops.KernelError, match="point 3"):
        Sampler.read(ids)
    # and a step afterwards is clean
    runner = runner_for(tmp_path, TINY_B, "bfloat16")
    a = runner.open("a")
    logits = runner.step([StepEntry(a, [1, 2, 3], [2])])
    assert torch.isfinite(logits).all()
    ops.raise_on_kernel_error()
