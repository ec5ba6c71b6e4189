"""bin/trace_run as a program: standard input in, ``done`` lines and .f32 files out."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tests import traces
from tests.plain import model as plain
from tests.tiny import TINY_B, make_model_dir, random_tokens, read_weights, sizes_of

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 6e-2)])
def test_trace_run_program(tmp_path, dtype, tol):
    tiny = TINY_B
    d = make_model_dir(tmp_path / "model", tiny)
    w = read_weights(d)
    reqs = {f"q{i}": random_tokens(n, tiny["cfg"].vocab_size, 50 + i) for i, n in enumerate([35, 48, 21, 66, 40])}
    ref = {rid: plain.forward(sizes_of(tiny["cfg"]), w, toks).numpy() for rid, toks in reqs.items()}
    steps = traces.mixed(reqs, seed=3)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(d), "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(traces.max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    V = tiny["cfg"].vocab_size

    def read_step(msg):
        f = out / f"{msg['step']}.f32"
        return np.fromfile(f, dtype="<f4").reshape(-1, V) if f.exists() else None

    got = traces.collect(read_step, steps)
    for (rid, pos), row in got.items():
        assert np.abs(row - ref[rid][pos]).max() < tol, (rid, pos)


def test_trace_run_writes_no_file_when_nothing_wanted(tmp_path):
    d = make_model_dir(tmp_path / "model", TINY_B)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out),
         "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert not (out / "0.f32").exists() and (out / "1.f32").exists()
