"""The Python entry point: token ids in, token ids out, through the engine.

``generate(model_dir, prompts, ...)`` in the manner of the reference's
``generate_cached`` (``acorninfer/generate.py:54-110``): prompts are lists of token ids, the
result lists contain the prompt followed by the generated ids, a generated eos id is
appended and then generation of that request stops.  Unlike the reference's helper,
which runs one request through a naive cache, all prompts run together through the paged
engine (continuous batching); the tokens are the same either way.
"""

from __future__ import annotations

from pathlib import Path

from .config.engine_config import EngineConfig
from .engine.engine import Engine
from .sampling.params import SamplingParams


def build_engine(model_dir: str | Path, *, dtype: str = "bfloat16", device: str = "cuda:0", num_blocks: int = 1024,
                 page_size: int = 16, max_running: int = 8, watermark_blocks: int = 8,
                 chunked_budget: int | None = None, warm_up: bool = False) -> Engine:
    """``warm_up``: run throw-away steps now (``ModelRunner.warm_up``) so that the first requests do not
    pay for kernels loaded and graphs captured at first use; worth it for an engine that serves."""
    cfg = EngineConfig(model_dir=str(model_dir), device=device, dtype=dtype, num_blocks=num_blocks,
                       page_size=page_size, max_running=max_running, watermark_blocks=watermark_blocks,
                       chunked_budget=chunked_budget)
    engine = Engine.from_config(cfg)
    if warm_up:
        engine.runner.warm_up()
    return engine


def generate_with_engine(engine: Engine, prompts: list[list[int]], *, max_new_tokens: int = 64,
                         temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, seed: int = 0,
                         eos_ids=None) -> list[list[int]]:
    """Runs all prompts to completion on an existing engine; returns prompt + generated ids each."""
    ids = [engine.submit(p, SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, seed=seed + i),
                         max_tokens=max_new_tokens, eos_ids=eos_ids) for i, p in enumerate(prompts)]
    while engine.has_pending():
        engine.step()
    out = [engine.seqs[i].all_ids for i in ids]
    for i in ids:
        engine.drop(i)
    return out


def generate(model_dir: str | Path, prompts: list[list[int]], *, max_new_tokens: int = 64, temperature: float = 0.0,
             top_p: float = 1.0, top_k: int = 0, seed: int = 0, eos_ids=None, **engine_options) -> list[list[int]]:
    """Loads the model folder, generates for every prompt, returns prompt + generated ids each.

    ``temperature == 0`` is greedy.  ``eos_ids`` None takes the model's own
    (``config.json``'s ``eos_token_id``); an empty collection never stops early.
    ``engine_options`` are those of :func:`build_engine`.
    """
    engine = build_engine(model_dir, **engine_options)
    out = generate_with_engine(engine, prompts, max_new_tokens=max_new_tokens, temperature=temperature,
                               top_p=top_p, top_k=top_k, seed=seed, eos_ids=eos_ids)
    engine.assert_balanced()
    return out
