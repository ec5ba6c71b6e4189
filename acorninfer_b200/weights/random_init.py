"""Random-weights mode: a model folder from a configuration and a seed.

Every tensor is drawn from a generator seeded by (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or in which order they are made.
Matrices are N(0, sigma), norm weights 1 + N(0, sigma_norm) (sigma_norm = 0 gives ones).
Values are rounded to the stored dtype (bfloat16 by default), so every reader of the
folder sees the same numbers.  The reference has no such mode: its tests take torch's
default initialisers under ``torch.manual_seed(0)`` (``tests/conftest.py:12-15``).
"""

from __future__ import annotations

import hashlib
from pathlib import Path

import torch

from ..config.model_config import ModelConfig, dump_config
from ..parts.base import TensorSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, spec: TensorSpec, seed: int, sigma: float, sigma_norm: float,
                  dtype: torch.dtype, device: torch.device | str = "cpu") -> torch.Tensor:
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(_tensor_seed(seed, name))
    if spec.init == "table":
        return torch.randint(0, 2 ** 15, spec.shape, generator=gen, device=device, dtype=torch.int32)
    if spec.init == "norm":
        t = torch.ones(spec.shape, dtype=torch.float32, device=device)
        if sigma_norm:
            t += sigma_norm * torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32)
        return t.to(dtype)
    if device.type == "cuda" and dtype != torch.float32:
        # Large matrices on the device: draw in the stored dtype to keep the peak small.
        return torch.randn(spec.shape, generator=gen, device=device, dtype=dtype).mul_(sigma)
    return (sigma * torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32)).to(dtype)


def random_state(expected: dict[str, TensorSpec], seed: int, sigma: float = 0.02, sigma_norm: float = 0.0,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device | str = "cpu") -> dict[str, torch.Tensor]:
    return {name: random_tensor(name, spec, seed, sigma, sigma_norm, dtype, device)
            for name, spec in expected.items() if not spec.optional}


def write_random_model(model_dir: str | Path, cfg: ModelConfig, seed: int, sigma: float = 0.02,
                       sigma_norm: float = 0.0, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Writes ``config.json`` and ``model.safetensors`` for ``cfg`` into ``model_dir``."""
    from ..models.decoder import expected_tensors
    from ..registry import spec_for

    model_dir = Path(model_dir)
    dump_config(cfg, model_dir)
    expected = expected_tensors(spec_for(cfg))
    tensors = random_state(expected, seed, sigma, sigma_norm, dtype, "cpu")
    write_safetensors(model_dir / "model.safetensors", tensors,
                      {"format": "pt", "seed": seed, "sigma": sigma, "sigma_norm": sigma_norm})
    return model_dir
