"""Random weights drawn on the device are the weights a folder written on the host holds."""

import pytest
import torch

from tests.tiny import TINY_B, TINY_D, make_model_dir, read_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tiny", [TINY_B, TINY_D], ids=["tiny_b", "tiny_d"])
def test_from_random_and_write_random_model_give_identical_tensors(tmp_path, tiny):
    from acorninfer_b200.models.decoder import expected_tensors
    from acorninfer_b200.registry import spec_for
    from acorninfer_b200.weights.random_init import random_state

    folder = read_weights(make_model_dir(tmp_path, tiny))
    expected = expected_tensors(spec_for(tiny["cfg"]))
    on_device = random_state(expected, tiny["seed"], tiny["sigma"], tiny["sigma_norm"], torch.bfloat16, "cuda:0")
    assert set(folder) == set(on_device)
    for name, t in folder.items():
        assert t.dtype == on_device[name].dtype == torch.bfloat16
        assert torch.equal(t, on_device[name].cpu()), name


def test_device_generator_matches_the_host_for_every_kind_and_offset():
    from acorninfer_b200.parts.base import TensorSpec
    from acorninfer_b200.weights.random_init import random_tensor

    for init, shape, dtype in (("matrix", (1000, 333), torch.bfloat16), ("matrix", (257, 129), torch.float32),
                               ("norm", (4096,), torch.bfloat16), ("norm", (333,), torch.float32),
                               ("table", (100, 9), torch.int32)):
        spec = TensorSpec(shape, init)
        host = random_tensor("t.weight", spec, 9, 0.02, 0.3, dtype, "cpu", backend="numpy")
        dev = random_tensor("t.weight", spec, 9, 0.02, 0.3, dtype, "cuda:0")
        assert torch.equal(host, dev.cpu()), (init, dtype)
        rows = random_tensor("t.weight", spec, 9, 0.02, 0.3, dtype, "cuda:0", rows=(50, 90))
        assert torch.equal(rows.cpu(), host[50:90])


def test_engines_from_a_folder_and_from_the_device_give_the_same_logits(tmp_path):
    from acorninfer_b200.engine.batch import StepEntry
    from acorninfer_b200.engine.runner import ModelRunner

    tiny = TINY_D
    d = make_model_dir(tmp_path, tiny)
    kw = dict(dtype="bfloat16", num_blocks=16, page_size=16, max_requests=2)
    a = ModelRunner.from_model_dir(d, **kw)
    b = ModelRunner.from_random(tiny["cfg"], tiny["seed"], tiny["sigma"], tiny["sigma_norm"], **kw)
    toks = list(range(3, 60))
    la = a.step([StepEntry(a.open("x"), toks, [len(toks) - 1])])
    lb = b.step([StepEntry(b.open("x"), toks, [len(toks) - 1])])
    assert torch.equal(la, lb)
