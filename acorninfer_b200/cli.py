"""``python -m acorninfer_b200``: the command line.

``generate`` has the reference's options with their names and meanings
(``acorninfer/cli.py:16-26``): ``--prompt``, ``--model-dir``, ``--max-new-tokens`` (64),
``--temperature`` (0 = greedy), ``--top-p``, ``--top-k`` (0 = disabled); and the engine's
(``acorninfer/bench.py:107-112``): ``--num-blocks``, ``--page-size``, ``--max-running``,
``--watermark-blocks``.  Added: ``--prompt-ids`` (comma-separated ids, no tokenizer
needed), ``--seed``, ``--dtype``, ``--chunked-budget``.
``random-model`` writes a model folder with seeded random weights from a config.json.
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def _add_engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--num-blocks", type=int, default=1024)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--max-running", type=int, default=8)
    p.add_argument("--watermark-blocks", type=int, default=8)
    p.add_argument("--chunked-budget", type=int, default=None, help="most tokens in one step (default: whole prompts)")


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="acorninfer_b200")
    sub = parser.add_subparsers(dest="cmd", required=True)
    gen = sub.add_parser("generate", help="greedy or sampled generation")
    gen.add_argument("--prompt", default=None, help="text prompt (needs tokenizer.json in the model folder)")
    gen.add_argument("--prompt-ids", default=None, help="comma-separated token ids instead of --prompt")
    gen.add_argument("--model-dir", required=True)
    gen.add_argument("--max-new-tokens", type=int, default=64)
    gen.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    gen.add_argument("--top-p", type=float, default=1.0)
    gen.add_argument("--top-k", type=int, default=0, help="0 = disabled")
    gen.add_argument("--seed", type=int, default=0)
    _add_engine_options(gen)
    rnd = sub.add_parser("random-model", help="write config.json + model.safetensors with seeded random weights")
    rnd.add_argument("--config", required=True, help="a config.json to take the sizes from")
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--sigma", type=float, default=0.02)
    rnd.add_argument("--sigma-norm", type=float, default=0.0)
    args = parser.parse_args(argv)

    if args.cmd == "random-model":
        from .registry import config_from_dict
        from .weights.random_init import write_random_model
        cfg = config_from_dict(json.loads(open(args.config).read()))
        print(write_random_model(args.out, cfg, args.seed, args.sigma, args.sigma_norm))
        return 0

    from .generation import build_engine, generate_with_engine

    if (args.prompt is None) == (args.prompt_ids is None):
        parser.error("give exactly one of --prompt and --prompt-ids")
    tok = None
    if args.prompt is not None:
        from .tokenizer import Tokenizer
        tok = Tokenizer(f"{args.model_dir}/tokenizer.json")
        prompt_ids = tok.encode(args.prompt)
    else:
        prompt_ids = [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    if not prompt_ids:
        raise SystemExit("prompt encoded to zero tokens; pass a non-empty prompt")

    t0 = time.perf_counter()
    engine = build_engine(args.model_dir, dtype=args.dtype, device=args.device, num_blocks=args.num_blocks,
                          page_size=args.page_size, max_running=args.max_running,
                          watermark_blocks=args.watermark_blocks, chunked_budget=args.chunked_budget)
    print(f"model loaded in {time.perf_counter() - t0:.1f}s", file=sys.stderr)
    t0 = time.perf_counter()
    ids = generate_with_engine(engine, [prompt_ids], max_new_tokens=args.max_new_tokens,
                               temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, seed=args.seed)[0]
    elapsed = time.perf_counter() - t0
    new = len(ids) - len(prompt_ids)
    print(tok.decode(ids) if tok is not None else ",".join(str(t) for t in ids))
    print(f"--- {new} tokens in {elapsed:.2f}s ({new / max(elapsed, 1e-9):.2f} tok/s)", file=sys.stderr)
    return 0
