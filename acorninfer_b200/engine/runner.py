"""The step function: one batch of (request, its next tokens) -> logits at the wanted places.

``ModelRunner`` owns the model, the cache manager and the step workspace.  ``step``
  1. validates the batch on the host (a bad batch raises; nothing ran, nothing is held),
  2. reserves the pages the step writes (all requests or none: ``PoolExhausted``),
  3. lays the batch out and uploads it in one transfer (a step whose arrays do not fit the
     workspace raises ``BatchError`` here; the pages of 2 are given back first),
  4. runs the model over exactly the tokens given, reading earlier tokens from the cache,
  5. commits the new lengths (windowed groups give pages back),
and returns float32 logits ``[wanted, vocab]`` in the order of the entries and their
``want`` lists.  Prompt portions and single decoded tokens are the same code path; how the
tokens were cut into steps, what else is in the batch and which pages hold them change the
result by rounding only.  Generation, replay and the benchmark all go through here.

Reference: the reference runs a scheduled step as up to four forwards
(``acorninfer/engine/engine.py:167-262``, ``acorninfer/engine/executor.py:21-108``);
here it is one forward over the flat token batch.
"""

from __future__ import annotations

from collections import OrderedDict
from pathlib import Path

import torch

from ..cache.manager import CacheManager, RequestCache
from ..cache.pools import PoolExhausted
from ..config.model_config import ModelConfig
from ..kernels import ops
from ..models.decoder import Decoder
from ..registry import load_config, spec_for
from ..weights.loader import load_tensors
from ..weights.random_init import random_state
from .batch import (PREFILL_GRAPH_MAX_TOKENS, BatchError, StepEntry, StepWorkspace, pad_decode_plan, pad_prefill_plan,
                    plan_step, prefill_bucket, prefill_buckets, validate_entries)

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


MAX_GRAPHS = 384


class ModelRunner:
    def __init__(self, config: ModelConfig, tensors: dict[str, torch.Tensor] | None, *, dtype: str = "bfloat16",
                 device: str = "cuda:0", num_blocks: int = 1024, page_size: int = 16, max_requests: int = 64,
                 max_step_tokens: int = 8192, decoder: Decoder | None = None, decode_graph: bool = True,
                 workspace_ints: int = 1 << 20):
        self.config = config
        self.dtype = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        self.device = torch.device(device)
        ops.lib()      # fails here, loudly, if there is no device or no compiled kernels
        torch.cuda.set_device(self.device)
        self.spec = spec_for(config)
        self.decoder = decoder or Decoder(self.spec, self.dtype, self.device, page_size)
        if tensors is not None:
            self.decoder.bind(tensors)
        kv_needs, state_needs = self.decoder.cache_needs()
        self.manager = CacheManager(kv_needs, state_needs, num_blocks, page_size, max_requests,
                                    dtype=self.dtype, device=self.device)
        self.caches = self.decoder.entry_caches(self.manager)
        self.max_step_tokens = max_step_tokens
        self.step_arrays = self.decoder.step_arrays()     # per-step arrays the parts' kernels read
        self.workspace = StepWorkspace(self.device, workspace_ints)
        self.vocab_size = self.spec.vocab_size
        # CUDA graphs of all-decode steps, keyed by the sizes that fix every launch of the step
        self.decode_graph = decode_graph and self.decoder.graph_safe
        # Padding a prompt portion writes keys and values for tokens that do not exist: harmless where a
        # request's next tokens overwrite them before they are read, which holds for caches that keep every
        # key; not for windows (pages are given back by position) nor for state that every token updates.
        self.prefill_graph = not self.manager.state_needs and all(g.window is None for g in self.manager.groups)
        self._graphs: OrderedDict[tuple, object] = OrderedDict()        # least recently replayed first
        self._graph_seen: OrderedDict[tuple, int] = OrderedDict()
        self._graph_pool = None
        self.graph_kernel_launches = 0
        self.graph_replays = 0

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_model_dir(cls, model_dir: str | Path, **kw) -> "ModelRunner":
        config = load_config(model_dir)
        dtype = kw.get("dtype", "bfloat16")
        tdtype = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        device = kw.get("device", "cuda:0")
        probe = Decoder(spec_for(config), tdtype, device, kw.get("page_size", 16))
        tensors = load_tensors(model_dir, probe.expected_tensors(), tdtype, device, probe.ignorable_tensors())
        probe.bind(tensors)
        return cls(config, None, decoder=probe, **kw)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int, sigma: float = 0.02, sigma_norm: float = 0.0,
                    **kw) -> "ModelRunner":
        """Random weights drawn straight on the device (no folder): for benchmarks of large sizes."""
        dtype = kw.get("dtype", "bfloat16")
        tdtype = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        device = kw.get("device", "cuda:0")
        probe = Decoder(spec_for(config), tdtype, device, kw.get("page_size", 16))
        tensors = random_state(probe.expected_tensors(), seed, sigma, sigma_norm, torch.bfloat16, device)
        if tdtype == torch.float32:
            tensors = {k: v.float() for k, v in tensors.items()}
        probe.bind(tensors)
        del tensors
        return cls(config, None, decoder=probe, **kw)

    # ------------------------------------------------------------------ requests

    def open(self, request_id) -> RequestCache:
        return self.manager.open(request_id)

    def close(self, cache: RequestCache) -> None:
        self.manager.close(cache)

    def warm_up(self, prompt_tokens: tuple[int, ...] = (16, 64, 128, 256, 512, 1024, 2048, 4096, 8192),
                decode_rows: tuple[int, ...] = (1, 2, 4, 8),
                decode_contexts: tuple[int, ...] = (200, 400, 800, 1600, 3200)) -> None:
        """Runs throw-away steps so that what a first request would pay for is paid at load: the
        library's kernels for prompt portions of several sizes (it loads them when first used), the
        captured graphs of short prompt portions (every bucket) and those of small all-decode steps at
        several context lengths.  Sizes the pools cannot hold are left out;
        every page and slot is given back."""
        free = min(self.manager.free_pages()) if self.manager.groups else 0
        page = self.manager.page_size
        for T in sorted(set(prompt_tokens)):
            if T > self.max_step_tokens or -(-T // page) > free or self.manager.slots.num_free < 1:
                continue
            rc = self.open(("warm-up", T))
            try:
                self.step([StepEntry(rc, [0] * T, [T - 1])])
            finally:
                self.close(rc)
        if self.decode_graph and self.prefill_graph:
            # a short prompt alone in its step replays a captured graph: seen, captured, replayed, per bucket
            for T in prefill_buckets():
                if T > self.max_step_tokens or -(-T // page) > free or self.manager.slots.num_free < 1:
                    continue
                for _ in range(3):
                    rc = self.open(("warm-up", "bucket", T))
                    try:
                        self.step([StepEntry(rc, [0] * T, [T - 1])])
                    finally:
                        self.close(rc)
        # all-decode steps: per row count, and per width of the block table (it doubles with the context:
        # requests that already hold 0, 200, 400, ... tokens, whose pages are taken but never written)
        for R in sorted(set(decode_rows)):
            for held in (0,) + tuple(decode_contexts):
                pages = -(-(held + 4) // page)
                if R > self.manager.slots.num_free or R * pages > min(self.manager.free_pages()):
                    continue
                rcs = [self.open(("warm-up", R, held, i)) for i in range(R)]
                try:
                    for rc in rcs:
                        if held:
                            self.manager.extend(rc, held)
                            self.manager.commit(rc, held)
                    for _ in range(4):                                    # the first token; then seen, captured, replayed
                        self.step([StepEntry(rc, [0], [0]) for rc in rcs])
                finally:
                    for rc in rcs:
                        self.close(rc)
        torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ the step

    def reserve(self, entries: list[StepEntry]) -> None:
        """Pages for every entry of the step, or for none of them."""
        need = [0] * len(self.manager.groups)
        for e in entries:
            for gi, n in enumerate(self.manager.pages_needed(e.cache, e.cache.length + len(e.tokens))):
                need[gi] += n
        free = self.manager.free_pages()
        for gi, (n, f) in enumerate(zip(need, free)):
            if n > f:
                raise PoolExhausted(f"step needs {n} page(s) in cache group {gi}, {f} free")
        for e in entries:
            self.manager.extend(e.cache, e.cache.length + len(e.tokens))

    @torch.inference_mode()
    def step(self, entries: list[StepEntry], device_tokens: torch.Tensor | None = None) -> torch.Tensor | None:
        """``device_tokens``: int32 ids on the device (the tokens the previous step sampled); entries
        with ``from_device`` take their id from there, so the host need not have read them yet."""
        validate_entries(entries, self.vocab_size, self.max_step_tokens)
        if device_tokens is None and any(e.from_device is not None for e in entries):
            raise BatchError("entries take ids from the device but no device_tokens were given")
        self.reserve(entries)
        try:
            plan = plan_step(entries, self.manager, self.step_arrays)
            self.last_plan = plan
            graph = self.decode_graph and plan.all_decode
            if graph:
                # padded to a bucket of row counts, so that a few captured graphs serve every batch size
                plan = pad_decode_plan(plan, self.manager.pad_pages, self.manager.pad_slot, self.step_arrays)
            elif (self.decode_graph and self.prefill_graph and plan.num_rows == 1
                  and plan.num_tokens <= PREFILL_GRAPH_MAX_TOKENS
                  and prefill_bucket(plan.num_tokens) <= self.max_step_tokens):
                # a short prompt portion alone in its step (a request that arrives at an idle engine): such
                # a step is bound by the host that launches it, so it is padded to a bucket of token counts
                # and replayed from a captured graph like the all-decode steps
                padded = pad_prefill_plan(plan, self.manager.pad_pages, self.manager.page_size, self.step_arrays)
                if self.workspace.layout(padded)[1] <= self.workspace.capacity:      # else: as it is, launch by launch
                    graph, plan = True, padded
            inputs = self.workspace.upload(plan)
        except Exception:
            for e in entries:           # nothing was launched: the step holds nothing
                self.manager.trim(e.cache)
            raise
        if plan.patch_dst.size:
            ops.patch_tokens(inputs.token_ids, inputs.patch_dst, inputs.patch_src, device_tokens)
        if graph:
            logits = self._decode_step(plan, inputs)
            if logits is not None and plan.num_logits != self.last_plan.num_logits:
                logits = logits[:self.last_plan.num_logits]
        else:
            logits = self.decoder.forward(inputs, self.caches)
        for e in entries:
            self.manager.commit(e.cache, e.cache.length + len(e.tokens))
        return logits

    # ------------------------------------------------------------------ captured decode steps

    def _decode_step(self, plan, inputs):
        """A step whose shape repeats (an all-decode step, or a short prompt portion alone, both padded to
        buckets): replayed from a CUDA graph once its shape has been seen twice.  At most ``MAX_GRAPHS``
        graphs are kept; the one replayed longest ago makes room for a new one.

        The step arrays were just uploaded to the addresses the graph reads (the address of every
        array the model reads is a function of the key), so a replay is this step.  The returned
        logits are the graph's output buffer: valid until the next step."""
        key = self.workspace.shape_key(plan)
        entry = self._graphs.get(key)
        if entry is not None:
            self._graphs.move_to_end(key)
            graph, logits, launches = entry
            graph.replay()
            self.graph_kernel_launches += launches
            self.graph_replays += 1
            return logits
        seen = self._graph_seen.pop(key, 0) + 1
        self._graph_seen[key] = seen
        if len(self._graph_seen) > 4 * MAX_GRAPHS:                       # shapes met once and never again
            self._graph_seen.popitem(last=False)
        logits = self.decoder.forward(inputs, self.caches)
        if seen >= 2:
            if len(self._graphs) >= MAX_GRAPHS:                          # the shape replayed longest ago makes room
                self._graphs.popitem(last=False)
            # Capturing launches nothing: the eager run above is this step's result (and the warm-up).
            before = ops.LAUNCHES
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                out = self.decoder.forward(inputs, self.caches)
            launches = ops.LAUNCHES - before
            ops.LAUNCHES = before
            self._graphs[key] = (graph, out, launches)
        return logits
