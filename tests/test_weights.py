"""Weights: the container, the dtype policy, the one error that lists everything wrong."""

import struct

import pytest
import torch

from acorninfer_b200.models.decoder import expected_tensors
from acorninfer_b200.registry import spec_for
from acorninfer_b200.weights.loader import load_tensors
from acorninfer_b200.weights.random_init import random_state, write_random_model
from acorninfer_b200.weights.safetensors_io import SafetensorsFile, WeightsError, write_safetensors
from tests.tiny import TINY_A, TINY_B, make_model_dir, read_weights


def test_container_round_trip_and_matches_the_safetensors_package(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64), "c": torch.randn(2, 2)}
    write_safetensors(tmp_path / "x.safetensors", t)
    f = SafetensorsFile(tmp_path / "x.safetensors")
    for k, v in t.items():
        assert torch.equal(f.tensor(k), v)
    from safetensors.torch import load_file
    other = load_file(str(tmp_path / "x.safetensors"))
    for k, v in t.items():
        assert torch.equal(other[k], v)


def test_random_model_is_reproducible_and_named_by_tensor(tmp_path):
    a = read_weights(make_model_dir(tmp_path / "a", TINY_A))
    b = read_weights(make_model_dir(tmp_path / "b", TINY_A))
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert "lm_head.weight" not in a                      # tied: no separate output matrix
    assert "lm_head.weight" in read_weights(make_model_dir(tmp_path / "c", TINY_B))
    norm = a["model.layers.0.input_layernorm.weight"].float()
    assert abs(norm.mean() - 1) < 0.1 and norm.std() > 0.02   # 1 + N(0, 0.1)
    assert all(v.dtype == torch.bfloat16 for v in a.values())
    # a tensor's values depend on (seed, name) only
    exp = expected_tensors(spec_for(TINY_A["cfg"]))
    one = random_state({"model.norm.weight": exp["model.norm.weight"]}, TINY_A["seed"], 0.02, 0.1)
    assert torch.equal(one["model.norm.weight"], a["model.norm.weight"])


def test_dtype_policy(tmp_path):
    d = make_model_dir(tmp_path / "m", TINY_A)
    exp = expected_tensors(spec_for(TINY_A["cfg"]))
    assert all(v.dtype == torch.bfloat16 for v in load_tensors(d, exp, torch.bfloat16, "cpu").values())
    assert all(v.dtype == torch.float32 for v in load_tensors(d, exp, torch.float32, "cpu").values())
    d32 = write_random_model(tmp_path / "m32", TINY_A["cfg"], 1, dtype=torch.float32)
    # stored in 32 bits: stays so, also under a bfloat16 engine
    assert all(v.dtype == torch.float32 for v in load_tensors(d32, exp, torch.bfloat16, "cpu").values())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model_dir(tmp_path / "m", TINY_B)
    w = read_weights(d)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.7.extra.weight"] = torch.zeros(2)
    w["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16, dtype=torch.bfloat16)
    write_safetensors(d / "model.safetensors", w)
    exp = expected_tensors(spec_for(TINY_B["cfg"]))
    with pytest.raises(WeightsError) as err:
        load_tensors(d, exp, torch.bfloat16, "cpu")
    msg = str(err.value)
    assert "missing (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected (1)" in msg and "model.layers.7.extra.weight" in msg
    assert "wrong shape (1)" in msg and "q_norm.weight: file has [16], model wants [32]" in msg


def test_tied_model_may_carry_a_copy_of_the_output_matrix(tmp_path):
    d = make_model_dir(tmp_path / "m", TINY_A)
    w = read_weights(d)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    write_safetensors(d / "model.safetensors", w)
    exp = expected_tensors(spec_for(TINY_A["cfg"]))
    load_tensors(d, exp, torch.bfloat16, "cpu", ignorable=("lm_head.weight",))
    with pytest.raises(WeightsError, match="unexpected"):
        load_tensors(d, exp, torch.bfloat16, "cpu")


def test_truncated_and_missing_files(tmp_path):
    with pytest.raises(WeightsError, match="neither"):
        load_tensors(tmp_path, {}, torch.bfloat16, "cpu")
    d = make_model_dir(tmp_path / "m", TINY_A)
    data = (d / "model.safetensors").read_bytes()
    (d / "model.safetensors").write_bytes(data[:len(data) // 2])
    with pytest.raises(WeightsError, match="truncated"):
        SafetensorsFile(d / "model.safetensors")
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 10 ** 12) + b"{}")
    with pytest.raises(WeightsError, match="header"):
        SafetensorsFile(d / "model.safetensors")


def test_sharded_folder_with_index(tmp_path):
    import json
    d = make_model_dir(tmp_path / "m", TINY_A)
    w = read_weights(d)
    names = sorted(w)
    half = len(names) // 2
    write_safetensors(d / "s1.safetensors", {n: w[n] for n in names[:half]})
    write_safetensors(d / "s2.safetensors", {n: w[n] for n in names[half:]})
    (d / "model.safetensors").unlink()
    (d / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}))
    got = load_tensors(d, expected_tensors(spec_for(TINY_A["cfg"])), torch.bfloat16, "cpu")
    assert all(torch.equal(got[n], w[n]) for n in names)


def test_counter_based_generator_three_ways_on_the_host():
    """The NumPy restatement of the formula, the compiled host loop and row ranges agree bit for bit;
    the values have the mean and spread asked for; tensors and seeds do not repeat each other."""
    import numpy as np
    from acorninfer_b200.parts.base import TensorSpec
    from acorninfer_b200.weights.random_init import normal_numpy, random_tensor, tensor_key

    for init, shape, dtype in (("matrix", (130, 77), torch.bfloat16), ("matrix", (9, 5, 3), torch.float32),
                               ("norm", (301,), torch.bfloat16), ("norm", (64,), torch.float32),
                               ("table", (7, 11), torch.int32)):
        spec = TensorSpec(shape, init)
        a = random_tensor("some.weight", spec, 17, 0.03, 0.2, dtype, "cpu", backend="numpy")
        b = random_tensor("some.weight", spec, 17, 0.03, 0.2, dtype, "cpu", backend="host")
        assert a.dtype == dtype and tuple(a.shape) == shape and torch.equal(a, b), (init, shape)
        part = random_tensor("some.weight", spec, 17, 0.03, 0.2, dtype, "cpu", rows=(2, 6), backend="numpy")
        assert torch.equal(part, a[2:6])
        other = random_tensor("other.weight", spec, 17, 0.03, 0.2, dtype, "cpu", backend="numpy")
        again = random_tensor("some.weight", spec, 18, 0.03, 0.2, dtype, "cpu", backend="numpy")
        assert not torch.equal(a, other) and not torch.equal(a, again)
    big = normal_numpy(tensor_key(3, "w"), 0, 200_000, 0.5, 0.0).astype(np.float64)
    assert abs(big.mean()) < 0.005 and abs(big.std() - 0.5) < 0.005
    assert abs(np.mean((big / big.std()) ** 4) - 2.85) < 0.05          # sum of eight uniforms: kurtosis 3 - 1.2 / 8
    ones = random_tensor("n.weight", TensorSpec((50,), "norm"), 1, 0.02, 0.0, torch.bfloat16, "cpu")
    assert torch.equal(ones, torch.ones(50, dtype=torch.bfloat16))


def test_a_part_can_register_an_init_kind_of_its_own():
    from acorninfer_b200.parts.base import TensorSpec
    from acorninfer_b200.weights.random_init import INIT_KINDS, random_state

    INIT_KINDS.register("test_decay", lambda d: torch.sigmoid(d.normal(1.0, 2.0).float()).to(d.dtype))
    try:
        t = random_state({"a.decay": TensorSpec((40,), "test_decay")}, 5, dtype=torch.float32)["a.decay"]
        assert t.shape == (40,) and float(t.min()) > 0 and float(t.max()) < 1 and float(t.mean()) > 0.7
    finally:
        INIT_KINDS._items.pop("test_decay")
    with pytest.raises(KeyError, match="unknown init kind 'nope'; known: matrix, norm, table"):
        random_state({"a": TensorSpec((4,), "nope")}, 5)
