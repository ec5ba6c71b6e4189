"""Weights by tensor name, checked against what the model expects.

The model says which tensors it expects (name -> shape); the folder says which it
has.  Every disagreement (missing, unexpected, wrong shape, unusable dtype) is
collected and reported in ONE error.  Dtype policy: floating tensors stored in 16
bits become bfloat16, tensors stored in 32-bit floats stay float32, integer tables
become int32; an engine running in float32 widens every floating tensor to float32
(exact).  The reference casts everything to one dtype (``acorninfer/weights.py:26``)
and leaves checking to ``load_state_dict(strict=True)`` (``acorninfer/models/qwen3.py:768``).
"""

from __future__ import annotations

from pathlib import Path
from typing import Iterable

import torch

from ..parts.base import TensorSpec
from .safetensors_io import SafetensorsFile, WeightsError, open_model_files

_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def target_dtype(stored: torch.dtype, init: str, engine_dtype: torch.dtype) -> torch.dtype:
    if init == "table" or stored in _INTS:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_names_and_shapes(expected: dict[str, TensorSpec], found: dict[str, tuple],
                           ignorable: Iterable[str] = (), where: str = "") -> None:
    """Raises one WeightsError that lists all missing, unexpected and mis-shaped tensors."""
    ignorable = set(ignorable)
    missing = [n for n, s in expected.items() if n not in found and not s.optional]
    unexpected = [n for n in found if n not in expected and n not in ignorable]
    wrong = [(n, found[n], expected[n].shape) for n in expected
             if n in found and tuple(found[n]) != tuple(expected[n].shape)]
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where or 'weights'}: tensors do not match the model"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(
            f"{n}: file has {list(got)}, model wants {list(want)}" for n, got, want in sorted(wrong)))
    raise WeightsError("\n".join(lines))


def load_tensors(model_dir: str | Path, expected: dict[str, TensorSpec], engine_dtype: torch.dtype,
                 device: torch.device | str, ignorable: Iterable[str] = ()) -> dict[str, torch.Tensor]:
    """Reads the expected tensors of a model folder onto ``device`` under the dtype policy."""
    files = open_model_files(model_dir)
    where: dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.entries:
            if name in where:
                raise WeightsError(f"{model_dir}: tensor '{name}' appears in {where[name].path.name} and {f.path.name}")
            where[name] = f
    check_names_and_shapes(expected, {n: f.entries[n].shape for n, f in where.items()}, ignorable, str(model_dir))
    bad = [f"{n} ({where[n].entries[n].dtype})" for n, s in expected.items()
           if n in where and s.init != "table" and where[n].entries[n].dtype not in _FLOATS]
    if bad:
        raise WeightsError(f"{model_dir}: tensors with a non-floating dtype where weights are expected: " + ", ".join(bad))
    out: dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if name not in where:
            continue
        t = where[name].tensor(name)
        out[name] = t.to(device=device, dtype=target_dtype(t.dtype, spec.init, engine_dtype))
    for f in files:
        f.close()
    return out
