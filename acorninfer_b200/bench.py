"""``python -m acorninfer_b200.bench``: throughput, time to first token and time per output
token of the engine under concurrent requests, in the manner of the reference's
``python -m acorninfer.bench`` (``acorninfer/bench.py:103-123``): the same options where it
has them (``--model-dir --device --num-blocks --page-size --max-running --watermark-blocks
--in-tokens --out-tokens --concurrency --seed``), seeded random prompts without eos ids
(``:40-47``), one short warm-up request that is not measured (``:154-159``), and one
``RESULT C=... ttft_p50=... tpot_mean=... tok_s=...`` line per concurrency level (``:68-99``).

Added: ``--random-config FILE`` (a config.json: random weights are drawn on the device, no
model folder needed) or ``--random-preset NAME`` (the sizes of a published model, e.g. qwen3-8b), ``--dtype``, ``--chunked-budget``, and ``--prompt-range LO HI`` /
``--output-range LO HI`` for requests of mixed lengths (the continuous-batching workload:
all requests arrive at once, prompts and outputs uniform in the ranges).  The engine warms its
kernels and decode graphs when it is built (``ModelRunner.warm_up``; ``--no-engine-warm-up`` leaves
that to the first requests, as the reference does).
"""

from __future__ import annotations

import argparse
import json
import statistics
import time

import torch

from .config.model_config import ModelConfig
from .config.presets import PRESETS, preset
from .engine.engine import Engine
from .engine.runner import ModelRunner
from .registry import config_from_dict
from .sampling.params import SamplingParams


def random_prompts(count: int, lengths: list[int], vocab: int, seed: int, avoid=()) -> list[list[int]]:
    """Seeded random prompts of the given lengths; ids in ``avoid`` (eos) are replaced."""
    gen = torch.Generator().manual_seed(seed)
    out = []
    for n in lengths[:count]:
        ids = torch.randint(0, vocab, (n,), generator=gen)
        for bad in avoid:
            if 0 <= bad < vocab:
                ids[ids == bad] = (bad + 1) % vocab
        out.append(ids.tolist())
    return out


def run_level(engine: Engine, prompts: list[list[int]], out_tokens: list[int]):
    """Submits everything at once, drives the engine until done, returns the request records."""
    sids = [engine.submit(p, SamplingParams(temperature=0.0), max_tokens=n, eos_ids=())
            for p, n in zip(prompts, out_tokens)]
    steps = 0
    while engine.has_pending():
        engine.step()
        steps += 1
    seqs = {sid: engine.seqs[sid] for sid in sids}
    for sid in sids:
        engine.drop(sid)
    engine.assert_balanced()
    return seqs, steps


def report(level: int, seqs: dict, steps: int) -> dict:
    ttfts = [s.first_token_at - s.created_at for s in seqs.values()]
    tpots = [(s.last_token_at - s.first_token_at) / (len(s.generated_ids) - 1)
             for s in seqs.values() if len(s.generated_ids) > 1]
    total = sum(len(s.generated_ids) for s in seqs.values())
    span = max(s.last_token_at for s in seqs.values()) - min(s.created_at for s in seqs.values())
    tpot = f"{statistics.mean(tpots) * 1000:.2f}ms" if tpots else "n/a"
    print(f"RESULT C={level} ttft_p50={statistics.median(ttfts):.4f}s ttft_mean={statistics.mean(ttfts):.4f}s "
          f"tpot_mean={tpot} tok_s={total / span:.2f} steps={steps} tokens={total} "
          f"preemptions={sum(s.preemptions for s in seqs.values())}")
    return {"concurrency": level, "ttft_p50": statistics.median(ttfts), "tok_s": total / span, "steps": steps}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="acorninfer_b200.bench", description=__doc__.split("\n\n")[0])
    p.add_argument("--model-dir", default=None)
    p.add_argument("--random-config", default=None, help="config.json to draw random weights for (no model folder)")
    p.add_argument("--random-preset", default=None, help="the same from a model's published sizes: " + ", ".join(sorted(PRESETS)))
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--num-blocks", type=int, default=1024)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--max-running", type=int, default=8)
    p.add_argument("--watermark-blocks", type=int, default=8)
    p.add_argument("--chunked-budget", type=int, default=None)
    p.add_argument("--in-tokens", type=int, default=128)
    p.add_argument("--out-tokens", type=int, default=32)
    p.add_argument("--prompt-range", type=int, nargs=2, default=None, metavar=("LO", "HI"))
    p.add_argument("--output-range", type=int, nargs=2, default=None, metavar=("LO", "HI"))
    p.add_argument("--concurrency", type=int, nargs="+", default=[1, 4, 8])
    p.add_argument("--seed", type=int, default=20261027)
    p.add_argument("--no-engine-warm-up", action="store_true", help="do not warm kernels and decode graphs at load")
    args = p.parse_args(argv)
    if sum(x is not None for x in (args.model_dir, args.random_config, args.random_preset)) != 1:
        p.error("give exactly one of --model-dir, --random-config and --random-preset")

    kw = dict(dtype=args.dtype, device=args.device, num_blocks=args.num_blocks, page_size=args.page_size,
              max_requests=args.max_running,
              max_step_tokens=max(8192, args.chunked_budget or 0, (args.prompt_range or [0, args.in_tokens])[1]))
    if args.model_dir is not None:
        print(f"loading {args.model_dir} -> {args.device} ({args.dtype}) ...")
        runner = ModelRunner.from_model_dir(args.model_dir, **kw)
    else:
        raw = preset(args.random_preset) if args.random_preset else json.loads(open(args.random_config).read())
        cfg: ModelConfig = config_from_dict(raw)
        print(f"random weights for {args.random_preset or args.random_config} -> {args.device} ({args.dtype}) ...")
        runner = ModelRunner.from_random(cfg, seed=args.seed, **kw)
    if not args.no_engine_warm_up:
        t0 = time.perf_counter()
        runner.warm_up(decode_rows=tuple(sorted({1, 2, 4, 8} | set(args.concurrency))))
        print(f"engine warm-up {time.perf_counter() - t0:.2f}s")
    engine = Engine(runner, max_running=args.max_running, watermark_blocks=args.watermark_blocks,
                    chunked_budget=args.chunked_budget, default_eos_ids=())
    vocab = runner.vocab_size
    eos = tuple(getattr(runner.config, "eos_token_id", ()))
    print(f"engine ready: num_blocks={args.num_blocks} page={args.page_size} max_running={args.max_running} "
          f"watermark={args.watermark_blocks} chunked_budget={args.chunked_budget}")

    run_level(engine, random_prompts(1, [8], vocab, args.seed, eos), [min(4, args.out_tokens)])
    print("warmup done (1 request, not measured)")
    results = []
    for level in args.concurrency:
        gen = torch.Generator().manual_seed(args.seed + level)
        if args.prompt_range:
            lens = torch.randint(args.prompt_range[0], args.prompt_range[1] + 1, (level,), generator=gen).tolist()
        else:
            lens = [args.in_tokens] * level
        if args.output_range:
            outs = torch.randint(args.output_range[0], args.output_range[1] + 1, (level,), generator=gen).tolist()
        else:
            outs = [args.out_tokens] * level
        t0 = time.perf_counter()
        seqs, steps = run_level(engine, random_prompts(level, lens, vocab, args.seed, eos), outs)
        results.append(report(level, seqs, steps))
        print(f"   wall {time.perf_counter() - t0:.3f}s, mean batch {sum(len(s.generated_ids) for s in seqs.values()) / max(steps, 1):.1f} tokens/step")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
