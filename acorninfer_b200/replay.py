"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and schedules nothing: every line of standard input is one step,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

whose entries run as one batch through the same :class:`ModelRunner` (model, step function,
cache manager, kernels) that generation uses.  For a step that wants logits, the float32
logits ``[wanted, vocab]`` (entries in order, then ``want`` in order) are written
little-endian to ``<out>/<step>.f32``.  After every step ``done <step>`` is printed and
flushed.  Requests named in ``end`` give back what they hold after the step.

``--max-tokens N`` sizes the page pool: N tokens, every live request's count rounded up to a
multiple of 64 (the page size divides 64), so that pages are reused as requests end.

The reference has no such program; its tests compare back ends under forced tokens
(``tests/test_forward_decode.py:86-99``), which is the idea this tool serves.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def parse_args(argv=None):
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder the <step>.f32 files are written to")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to 64)")
    p.add_argument("--page-size", type=int, default=16, help="tokens per cache page (divides 64)")
    p.add_argument("--device", default="cuda:0")
    return p.parse_args(argv)


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.page_size < 1 or 64 % args.page_size:
        print(f"trace_run: --page-size must divide 64, got {args.page_size}", file=sys.stderr)
        return 2
    if args.max_tokens < 1:
        print("trace_run: --max-tokens must be >= 1", file=sys.stderr)
        return 2
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)

    from .engine.runner import ModelRunner

    num_blocks = -(-args.max_tokens // args.page_size)
    runner = ModelRunner.from_model_dir(
        args.model, dtype=args.dtype, device=args.device, num_blocks=num_blocks, page_size=args.page_size,
        max_requests=16, max_step_tokens=max(args.max_tokens, 64))
    session = TraceSession(runner)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        logits = session.step(msg)
        if logits is not None:
            logits.astype("<f4", copy=False).tofile(out_dir / f"{msg['step']}.f32")
        print(f"done {msg['step']}", flush=True)
    return 0


class TraceSession:
    """Replays trace steps on a ModelRunner: opens a request at its first entry, runs each
    step's entries as one batch, closes the requests a step ends."""

    def __init__(self, runner):
        self.runner = runner
        self.live: dict[str, object] = {}

    def step(self, msg: dict):
        """Runs one step; returns the wanted logits as a float32 numpy array [wanted, vocab], or None."""
        import torch

        from .engine.batch import StepEntry
        from .kernels import ops

        entries = []
        for e in msg.get("entries", []):
            rid = str(e["id"])
            if rid not in self.live:
                self.live[rid] = self.runner.open(rid)
            entries.append(StepEntry(self.live[rid], [int(t) for t in e["tokens"]],
                                     [int(w) for w in e.get("want", [])]))
        out = None
        if entries:
            logits = self.runner.step(entries)
            if logits is not None:
                out = logits.detach().to("cpu", torch.float32).contiguous().numpy()
                ops.raise_on_kernel_error()     # the copy waited for the step: a kernel that gave up has said so
        for rid in msg.get("end", []):
            rc = self.live.pop(str(rid), None)
            if rc is not None:
                self.runner.close(rc)
        return out


if __name__ == "__main__":
    raise SystemExit(main())
