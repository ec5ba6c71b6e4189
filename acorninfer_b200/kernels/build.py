"""Compiles the CUDA sources under ``csrc/`` for sm_100a into one shared library.

The library is built in-tree (``csrc/_build/libacorn_kernels.so``) with nvcc, one
object per source in parallel, and is rebuilt when a source or header changes.  If
the tree is not writable the build goes to a per-user folder under the system's
temporary directory.  Progress lines go to stderr, since a first call may take a
minute.  There is no fallback: without nvcc and without a built library the import
of the kernels fails with the reason.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libacorn_kernels.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


class KernelBuildError(RuntimeError):
    pass


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _nvcc() -> str:
    for cand in (os.environ.get("ACORN_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise KernelBuildError("nvcc not found (PATH, /usr/local/cuda/bin): the CUDA kernels cannot be compiled")


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    override = os.environ.get("ACORN_BUILD_DIR")
    if override:
        return Path(override)
    local = CSRC / "_build"
    if _writable_dir(local):
        return local
    return Path(tempfile.gettempdir()) / f"acorninfer_b200-{os.getuid()}" / "_build"


def _log(msg: str) -> None:
    print(f"[acorninfer_b200] {msg}", file=sys.stderr, flush=True)


def ensure_built(verbose: bool = True) -> Path:
    """Returns the path of an up-to-date library, compiling what is stale.  ``ACORN_KERNEL_LIB`` names
    a library file to load as it is (a build with other compiler flags, for experiments)."""
    given = os.environ.get("ACORN_KERNEL_LIB")
    if given:
        if not Path(given).is_file():
            raise KernelBuildError(f"ACORN_KERNEL_LIB names {given}, which is not a file")
        return Path(given)
    digest = _digest()
    for cand in (CSRC / "_build", build_dir()):
        stamp, lib = cand / "stamp.txt", cand / LIB_NAME
        if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
            return lib
    out = build_dir()
    if not _writable_dir(out):
        raise KernelBuildError(f"cannot write the build folder {out}")
    nvcc = _nvcc()
    srcs = sources()
    if verbose:
        _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {out} ...")
    t0 = time.time()

    def compile_one(src: Path) -> Path:
        obj = out / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            _log(f"  compiled {src.name} ({time.time() - t0:.0f}s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp_lib = out / (LIB_NAME + f".tmp{os.getpid()}")
    cmd = [nvcc, "-shared", "-o", str(tmp_lib), *[str(o) for o in objs]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise KernelBuildError(f"linking {LIB_NAME} failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp_lib, out / LIB_NAME)
    (out / "stamp.txt").write_text(digest + "\n")
    if verbose:
        _log(f"built {LIB_NAME} in {time.time() - t0:.0f}s")
    return out / LIB_NAME


if __name__ == "__main__":
    print(ensure_built())
