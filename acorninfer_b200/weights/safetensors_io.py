"""Reading and writing the safetensors container, by tensor name.

Format: 8 bytes little-endian header length N, N bytes of JSON mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to
the end of the header; ``__metadata__`` is free text), then the raw little-endian
data.  The file is memory-mapped; a tensor is a view into the map until it is
copied to the device.

The reference loads through the ``safetensors`` package and needs
``model.safetensors.index.json`` (``acorninfer/weights.py:12-26``); its sharded
loader also takes a single ``model.safetensors`` (``acorninfer/weights.py:46-54``).
Both layouts are read here.
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from dataclasses import dataclass
from pathlib import Path

import torch


class WeightsError(ValueError):
    """A model folder whose tensors cannot be used: says which and why."""


_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    file: Path
    begin: int      # absolute byte offsets in the file
    end: int


class SafetensorsFile:
    """One open, memory-mapped safetensors file."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except OSError as exc:
            raise WeightsError(f"{self.path}: cannot open ({exc.strerror})") from None
        size = self.path.stat().st_size
        if size < 8:
            raise WeightsError(f"{self.path}: truncated (no header length)")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise WeightsError(f"{self.path}: truncated or corrupt header (length {hlen}, file {size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise WeightsError(f"{self.path}: header is not valid JSON ({exc})") from None
        base = 8 + hlen
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            dt = info.get("dtype")
            if dt not in _DTYPES:
                raise WeightsError(f"{self.path}: tensor '{name}' has unsupported dtype {dt!r}")
            dtype, width = _DTYPES[dt]
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(o) for o in info["data_offsets"])
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * width:
                raise WeightsError(
                    f"{self.path}: tensor '{name}' has {end - begin} bytes, shape {list(shape)} "
                    f"of {dt} needs {count * width}")
            if base + end > size:
                raise WeightsError(
                    f"{self.path}: truncated: tensor '{name}' ends at byte {base + end}, file has {size}")
            self.entries[name] = TensorEntry(name, dtype, shape, self.path, base + begin, base + end)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped bytes (read-only: copy before writing)."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # the map is read-only; tensors are copied before use
            flat = torch.frombuffer(memoryview(self._map)[e.begin:e.end], dtype=e.dtype)
        return flat.view(e.shape)

    def close(self) -> None:
        # Tensors handed out may still view the map: leave unmapping to the collector.
        self._fh.close()


def open_model_files(model_dir: str | Path) -> list[SafetensorsFile]:
    """The safetensors files of a model folder: the index's shards, else ``model.safetensors``."""
    model_dir = Path(model_dir)
    index = model_dir / "model.safetensors.index.json"
    if index.is_file():
        try:
            weight_map = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError) as exc:
            raise WeightsError(f"{index}: not a valid index ({exc})") from None
        return [SafetensorsFile(model_dir / shard) for shard in sorted(set(weight_map.values()))]
    single = model_dir / "model.safetensors"
    if single.is_file():
        return [SafetensorsFile(single)]
    raise WeightsError(f"{model_dir}: neither model.safetensors.index.json nor model.safetensors found")


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Writes CPU tensors to one file, in the order given."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise WeightsError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name, t in tensors.items():
            c = t.detach().contiguous().cpu()
            if c.numel():
                fh.write(c.view(torch.uint8).numpy().tobytes() if c.dim() else c.reshape(1).view(torch.uint8).numpy().tobytes())
