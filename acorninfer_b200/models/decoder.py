"""The generic decoder: parts built from a ModelSpec, run in the order its schedule says.

``forward`` is the whole model for one step: token table -> float32 residual stream ->
the scheduled layer runs -> final norm on the rows whose logits are wanted -> output
matrix -> float32 logits, with the spec's stages (if it names any) after the token table and
around the output matrix.  Reference for the order of operations:
``Qwen3ForCausalLM.forward`` in ``acorninfer/models/qwen3.py:491-518``.  The layer loop is a
loop over data: ``spec.schedule`` may name a layer twice, and a run may read the cache
of an earlier run instead of keeping its own.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in part kinds)
from ..kernels import ops
from ..parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, STAGES, BuildContext, KVNeeds,
                          ModelSpec, StateNeeds, TensorSpec, build_part)


@dataclass
class EntryCache:
    """What a schedule entry's mixer gets: the pages (its own or another run's), the cache
    group they belong to, whether this run writes them, and its state tensor if any."""

    entry: int
    group: int | None
    k_pages: torch.Tensor | None
    v_pages: torch.Tensor | None
    write: bool
    state: torch.Tensor | None


class Decoder:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, page_size: int = 16):
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.ctx = BuildContext(dtype=dtype, device=self.device, page_size=page_size)
        for name, ps in spec.positions.items():
            self.ctx.positions[name] = build_part(POSITION_ENCODINGS, ps, self.ctx)
        self.blocks = []
        self._named_parts: list[tuple[str, object]] = []     # (prefix, part) for tensor collection
        for ls in spec.layers:
            mixer = build_part(MIXERS, ls.mixer, self.ctx)
            ff = build_part(FEED_FORWARDS, ls.feed_forward, self.ctx)
            norms = {k: build_part(NORMS, v, self.ctx) for k, v in ls.norms.items()}
            block = BLOCKS.get(ls.block.kind)(ctx=self.ctx, mixer=mixer, feed_forward=ff, norms=norms,
                                              **ls.block.params)
            self.blocks.append(block)
            self._named_parts.append((ls.mixer.prefix, mixer))
            self._named_parts.append((ls.feed_forward.prefix, ff))
            for k, v in ls.norms.items():
                self._named_parts.append((v.prefix, norms[k]))
            self._named_parts.append((ls.block.prefix, block))
        self.final_norm = build_part(NORMS, spec.final_norm, self.ctx)
        self._named_parts.append((spec.final_norm.prefix, self.final_norm))
        self.stages = {}
        for where in ("after_embedding", "before_head", "after_head"):
            self.stages[where] = [build_part(STAGES, ps, self.ctx) for ps in getattr(spec, where)]
            self._named_parts.extend((ps.prefix, st) for ps, st in zip(getattr(spec, where), self.stages[where]))
        for i, e in enumerate(spec.schedule):
            if not (0 <= e.layer < len(spec.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}; the model has {len(spec.layers)}")
            if e.reads_cache_of is not None and not (0 <= e.reads_cache_of < i):
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, which is not earlier")
            if e.reads_cache_of is not None and spec.schedule[e.reads_cache_of].reads_cache_of is not None:
                raise ValueError(f"schedule entry {i} reads the cache of an entry that has none of its own")
        self.embedding: torch.Tensor | None = None
        self.head: torch.Tensor | None = None

    # ------------------------------------------------------------------ tensors

    def expected_tensors(self) -> dict[str, TensorSpec]:
        out: dict[str, TensorSpec] = {}
        s = self.spec
        out[s.embedding] = TensorSpec((s.vocab_size, s.hidden_size))
        for prefix, part in self._named_parts:
            for rel, ts in part.tensor_specs().items():
                out[prefix + rel] = ts
        if s.head is not None:
            out[s.head] = TensorSpec((s.vocab_size, s.hidden_size))
        return out

    def ignorable_tensors(self) -> tuple[str, ...]:
        # A tied model's file may still carry a copy of the output matrix.
        return ("lm_head.weight",) if self.spec.head is None else ()

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[s.embedding].contiguous()
        self.head = tensors[s.head].contiguous() if s.head is not None else self.embedding
        for prefix, part in self._named_parts:
            part.bind({rel: tensors[prefix + rel] for rel in part.tensor_specs() if prefix + rel in tensors})

    # ------------------------------------------------------------------ cache needs

    def cache_needs(self) -> tuple[dict[int, KVNeeds], dict[int, StateNeeds]]:
        """Per schedule entry that keeps something: its KV needs and its state needs."""
        kv: dict[int, KVNeeds] = {}
        state: dict[int, StateNeeds] = {}
        for i, e in enumerate(self.spec.schedule):
            needs = self.blocks[e.layer].mixer.cache_needs()
            if e.reads_cache_of is not None:
                owner = self.blocks[self.spec.schedule[e.reads_cache_of].layer].mixer.cache_needs()
                if needs.kv is None or owner.kv is None or needs.kv.group_key != owner.kv.group_key:
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {e.reads_cache_of}: "
                                     "their mixers keep different things")
                continue
            if needs.kv is not None:
                kv[i] = needs.kv
            if needs.state is not None:
                state[i] = needs.state
        return kv, state

    def entry_caches(self, manager) -> list[EntryCache]:
        out = []
        for i, e in enumerate(self.spec.schedule):
            owner = i if e.reads_cache_of is None else e.reads_cache_of
            if owner in manager.entry_group:
                k, v = manager.kv_pages(owner)
                group = manager.group_of(owner)
            else:
                k = v = group = None
            out.append(EntryCache(i, group, k, v, e.reads_cache_of is None, manager.state.get(i)))
        return out

    def step_arrays(self) -> dict:
        """The per-step arrays all parts declare (``Part.step_arrays``), by name."""
        out: dict = {}
        for _, part in self._named_parts:
            for name, build in part.step_arrays().items():
                out.setdefault(name, build)
        return out

    @property
    def graph_safe(self) -> bool:
        """Every part allows a step to be captured and replayed (see ``Part.graph_safe``)."""
        return all(getattr(part, "graph_safe", False) for _, part in self._named_parts)

    # ------------------------------------------------------------------ forward

    def forward(self, inputs, caches: list[EntryCache]) -> torch.Tensor | None:
        """Runs the step's tokens; returns float32 logits [wanted, vocab] (None if none wanted)."""
        resid32 = ops.embed(inputs.token_ids, self.embedding)
        for stage in self.stages["after_embedding"]:
            resid32 = stage.forward(resid32, inputs)
        delta = None
        sched = self.spec.schedule
        for i, e in enumerate(sched):
            # the norm that consumes this run's output: the next run's first norm (the final norm
            # works on selected rows only and keeps its own kernel)
            nxt = self.blocks[sched[i + 1].layer].first_norm(inputs.num_tokens) if i + 1 < len(sched) else None
            resid32, delta = self.blocks[e.layer].forward(resid32, delta, inputs, caches[i], next_norm=nxt)
        if inputs.num_logits == 0:
            return None
        h = self.final_norm.add_forward(resid32, delta, rows=inputs.logit_tokens)
        for stage in self.stages["before_head"]:
            h = stage.forward(h, inputs)
        logits = ops.linear(h, self.head, out_dtype=torch.float32)
        for stage in self.stages["after_head"]:
            logits = stage.forward(logits, inputs)
        return logits


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """The checkpoint tensors a model of this spec expects (no device needed)."""
    return Decoder(spec, torch.float32, "cpu").expected_tensors()
