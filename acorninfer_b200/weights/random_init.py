"""Random-weights mode: a model folder, or a model on the device, from a configuration and a seed.

Every element of every tensor is a function of (seed, tensor name, element index) alone: a
counter-based generator in integer arithmetic with one float32 multiplication (formula in
``csrc/random_fill.cu``, restated in NumPy below).  So a tensor's values do not depend on which
other tensors exist, in which order or on which device they are made, and any row range of a
tensor can be drawn without the rest: ``write_random_model`` on the host and
``ModelRunner.from_random`` on the device give bit-identical tensors for one seed, and a test can
draw the rows it needs of a model too large to hold twice.

How a tensor is filled is named by ``TensorSpec.init`` and looked up in ``INIT_KINDS``:
``matrix`` N(0, sigma), ``norm`` 1 + N(0, sigma_norm) (sigma_norm = 0 gives ones), ``table``
integers below 2^15.  A part whose parameters want another distribution registers its own kind:
a function of a :class:`Draw`, which offers the counter-based primitives.

The reference has no such mode: its tests take torch's default initialisers under
``torch.manual_seed(0)`` (``tests/conftest.py:12-15``), one model shared by oracle and engine.
"""

from __future__ import annotations

import ctypes
import hashlib
import math
import os
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..config.model_config import ModelConfig, dump_config
from ..parts.base import Registry, TensorSpec
from .safetensors_io import write_safetensors

_MASK = (1 << 64) - 1
_UNIT = 1.0 / (65536.0 * math.sqrt(2.0 / 3.0))      # 1 / standard deviation of the sum of eight 16-bit lanes


def tensor_key(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def _splitmix64(z: np.ndarray) -> np.ndarray:
    z = z + np.uint64(0x9E3779B97F4A7C15)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def lane_sums_numpy(key: int, first: int, count: int) -> tuple[np.ndarray, np.ndarray]:
    """(centred lane sums as int32, first hash as uint64) of elements first .. first + count - 1."""
    with np.errstate(over="ignore"):
        i = np.arange(first, first + count, dtype=np.uint64)
        base = np.uint64(key) + np.uint64(2) * i
        h0, h1 = _splitmix64(base), _splitmix64(base + np.uint64(1))
    s = np.zeros(count, np.int64)
    for lane in range(4):
        sh = np.uint64(16 * lane)
        s += ((h0 >> sh) & np.uint64(0xFFFF)).astype(np.int64) + ((h1 >> sh) & np.uint64(0xFFFF)).astype(np.int64)
    return (s - 4 * 65535).astype(np.int32), h0


def normal_numpy(key: int, first: int, count: int, sigma: float, mean: float = 0.0) -> np.ndarray:
    """float32 values ``mean + N(0, sigma)`` of the counter-based generator: the definition the
    compiled host loop and the device kernel are tested against."""
    s, _ = lane_sums_numpy(key, first, count)
    v = s.astype(np.float32) * np.float32(sigma * _UNIT)
    if mean != 0.0:
        v = np.float32(mean) + v
    return v.astype(np.float32)


_KIND_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 2}
_host_lib = None


def _host_library():
    """The compiled kernels' library for its host loop, or False if it cannot be had here."""
    global _host_lib
    if _host_lib is None:
        try:
            from ..kernels.build import ensure_built
            lib = ctypes.CDLL(str(ensure_built(verbose=False)))
            lib.acorn_random_fill_host.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint64, ctypes.c_uint64,
                                                   ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_int]
            lib.acorn_random_fill_host.restype = ctypes.c_int
            _host_lib = lib
        except Exception:
            _host_lib = False
    return _host_lib


def _fill(key: int, first: int, count: int, scale: float, mean: float, dtype: torch.dtype, device: torch.device,
          backend: str | None = None) -> torch.Tensor:
    """``count`` elements from element ``first`` on, flat.  ``backend``: None (device kernel on a CUDA
    device; on the host the compiled loop for large tensors, NumPy otherwise), "numpy" or "host"."""
    code = _KIND_CODE[dtype]
    scale32 = float(np.float32(scale * _UNIT))
    if device.type == "cuda":
        from ..kernels import ops
        out = torch.empty(count, dtype=dtype, device=device)
        ops.random_fill(out, key, first, scale32, float(mean), code)
        return out
    lib = _host_library() if backend == "host" or (backend is None and count >= 1 << 16) else False
    if backend == "host" and not lib:
        raise RuntimeError("the compiled host loop is not available")
    if lib:
        out = torch.empty(count, dtype=dtype)
        code_ = lib.acorn_random_fill_host(out.data_ptr(), count, key, first, scale32, float(mean), code,
                                           min(16, os.cpu_count() or 1))
        if code_ != 0:
            raise RuntimeError(f"acorn_random_fill_host failed with {code_}")
        return out
    if code == 2:
        return torch.from_numpy((lane_sums_numpy(key, first, count)[1] & np.uint64(0x7FFF)).astype(np.int32))
    s, _ = lane_sums_numpy(key, first, count)
    v = s.astype(np.float32) * np.float32(scale32)
    if mean != 0.0:
        v = (np.float32(mean) + v).astype(np.float32)
    return torch.from_numpy(v).to(dtype)             # bfloat16: round to nearest even


@dataclass
class Draw:
    """What an init kind gets: the tensor's name, shape and target, the mode's two scales, and the
    counter-based primitives.  ``rows``: (start, stop) of the leading dimension to draw, or None."""

    name: str
    shape: tuple[int, ...]
    seed: int
    sigma: float
    sigma_norm: float
    dtype: torch.dtype
    device: torch.device
    rows: tuple[int, int] | None = None
    backend: str | None = None

    def _range(self) -> tuple[int, int, tuple[int, ...]]:
        inner = int(np.prod(self.shape[1:])) if len(self.shape) > 1 else 1
        if self.rows is None:
            return 0, int(np.prod(self.shape)), tuple(self.shape)
        a, b = self.rows
        if not (0 <= a <= b <= self.shape[0]):
            raise ValueError(f"rows {self.rows} outside a leading dimension of {self.shape[0]}")
        return a * inner, (b - a) * inner, (b - a, *self.shape[1:])

    def normal(self, sigma: float, mean: float = 0.0, stream: str = "") -> torch.Tensor:
        """``mean + N(0, sigma)`` in the tensor's dtype; ``stream`` names a further independent
        draw of the same shape for kinds that need more than one."""
        first, count, shape = self._range()
        return _fill(tensor_key(self.seed, self.name + stream), first, count, sigma, mean, self.dtype, self.device,
                     self.backend).view(shape)

    def integers(self) -> torch.Tensor:
        first, count, shape = self._range()
        return _fill(tensor_key(self.seed, self.name), first, count, 0.0, 0.0, torch.int32, self.device,
                     self.backend).view(shape)


INIT_KINDS = Registry("init kind")
INIT_KINDS.register("matrix", lambda d: d.normal(d.sigma))
INIT_KINDS.register("norm", lambda d: d.normal(d.sigma_norm, 1.0))
INIT_KINDS.register("table", lambda d: d.integers())


def random_tensor(name: str, spec: TensorSpec, seed: int, sigma: float, sigma_norm: float,
                  dtype: torch.dtype, device: torch.device | str = "cpu", rows: tuple[int, int] | None = None,
                  backend: str | None = None) -> torch.Tensor:
    """The tensor ``name`` of the model with this seed (or rows ``rows[0]..rows[1]-1`` of it)."""
    return INIT_KINDS.get(spec.init)(Draw(name, tuple(spec.shape), seed, sigma, sigma_norm, dtype,
                                          torch.device(device), rows, backend))


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
