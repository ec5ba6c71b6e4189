"""Interfaces of the parts a layer is put together from, and their registries.

A model is data: a :class:`ModelSpec` lists layers, each layer names its parts by
*kind* (a registry key) with the sizes and constants as parameters, and a schedule
says in which order layers run.  A part never learns which model it is in: it gets
its parameters, a :class:`BuildContext` (dtype, device, page size, the shared
position encodings) and, at run time, the step's :class:`StepInputs` and the cache
handle of the schedule entry it runs for.

Interfaces
----------
``Norm``              ``forward(x32) -> x``; ``add_forward(resid32, delta) -> x`` (updates resid32)
``PositionEncoding``  constants for the mixers' kernels; ``apply(q, k, positions)`` for use alone
``Mixer``             ``cache_needs()``; ``forward(x, inputs, cache) -> delta``
``FeedForward``       ``forward(x, inputs) -> delta``
``Block``             ``forward(resid32, delta, inputs, cache) -> (resid32, delta)``
``Stage``             ``forward(x, inputs) -> x`` outside the layers (after the token table, around the head)

All activations are ``[tokens, width]`` over the flat token dimension of one step.
The residual stream is kept in float32 (``resid32``); what a part adds to it
(``delta``) is in the engine's activation dtype.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


# --------------------------------------------------------------------------- specs


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part expects.

    ``init`` tells the random-weights mode how to fill it: ``"matrix"`` N(0, sigma),
    ``"norm"`` 1 + N(0, sigma_norm), ``"table"`` integers.
    """

    shape: tuple[int, ...]
    init: str = "matrix"
    optional: bool = False


@dataclass(frozen=True)
class PartSpec:
    """A part by kind: the registry key, its sizes/constants, its weight-name prefix."""

    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (``block``) and the parts it arranges."""

    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: dict[str, PartSpec]


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers`` and may appear in
    several entries.  ``reads_cache_of`` names an earlier entry whose cache this run
    reads instead of writing one of its own."""

    layer: int
    reads_cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    embedding: str                      # tensor name of the token table [vocab, hidden]
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: str | None                    # tensor name of the output matrix; None: tied to embedding
    positions: dict[str, PartSpec] = field(default_factory=dict)   # shared position encodings by name
    # Stages outside the layers (kinds of the STAGES registry), applied in order; empty for a model
    # that goes from the token table straight into its layers and from the output matrix to logits.
    after_embedding: tuple[PartSpec, ...] = ()    # on the float32 residual stream [tokens, hidden]
    before_head: tuple[PartSpec, ...] = ()        # on the normed rows whose logits are wanted [wanted, hidden]
    after_head: tuple[PartSpec, ...] = ()         # on the float32 logits [wanted, vocab]


@dataclass
class BuildContext:
    dtype: torch.dtype
    device: torch.device
    page_size: int
    positions: dict[str, "PositionEncoding"] = field(default_factory=dict)


# --------------------------------------------------------------------------- cache needs


@dataclass(frozen=True)
class KVNeeds:
    """Keys and values in pages.  ``window`` None: every earlier key is read;
    an integer w: a query at position p reads keys p-w+1 .. p.  ``dtype`` None: the engine's
    activation dtype."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    dtype: torch.dtype | None = None

    @property
    def group_key(self) -> tuple:
        return ("kv", self.num_kv_heads, self.head_dim, self.window, self.dtype)


@dataclass(frozen=True)
class StateNeeds:
    """Per-request state of fixed size, kept in a slot of the slot pool (float32 unless
    ``dtype`` says otherwise)."""

    shape: tuple[int, ...]
    dtype: torch.dtype | None = None


@dataclass(frozen=True)
class CacheNeeds:
    kv: KVNeeds | None = None
    state: StateNeeds | None = None


# --------------------------------------------------------------------------- parts


class Part:
    """Base of all parts: declares checkpoint tensors and takes them when loaded.

    ``graph_safe``: the part's ``forward`` only launches work whose shape follows from the
    step's sizes (token count, row count, table stride) and reads everything else from device
    arrays, so a step may be captured once in a CUDA graph and replayed for other steps of the
    same sizes.  A part that looks at host-side values of the step leaves it False.
    """

    graph_safe = False

    def tensor_specs(self) -> dict[str, TensorSpec]:
        """Tensor names (relative to the part's prefix) -> spec."""
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receives the loaded tensors (same relative names) on the device."""

    def step_arrays(self) -> dict[str, Callable]:
        """Per-step int32 arrays this part's kernels read beside the common ones: name ->
        builder ``StepPlan -> numpy int32 array`` (any shape).  The step layer builds them on the
        host for every step, uploads them with the step's other arrays in the same transfer and
        hands them over as ``inputs.extra[name]`` (device view of the same shape) and
        ``inputs.plan.extra[name]`` (host).  Names are global to the model: parts that give the
        same name must mean the same array (it is built once).  For a captured step to be
        replayable a builder's output *shape* must follow from the step's sizes (tokens, rows,
        wanted logits, table strides); an all-decode step is built on the plan padded to its
        bucket."""
        return {}


class Norm(Part):
    def forward(self, x32: torch.Tensor, out: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        """The norm of ``x32``; with ``rows`` (int32 indices on the device) of those rows only."""
        raise NotImplementedError

    def as_epilogue(self, resid32: torch.Tensor):
        """An epilogue object with which the matrix product before this norm adds its result to
        the residual stream and hands on rows that only lack their RMS factor, or None if this
        norm cannot be fused that way."""
        return None

    def add_forward(self, resid32: torch.Tensor, delta: torch.Tensor | None,
                    out: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> torch.Tensor:
        """resid32 += delta (in place, float32), then the norm of it.  With ``rows`` the norm of
        ``resid32 + delta`` on those rows only, and the residual stream is left as it is."""
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Mixer(Part):
    # True: ``forward`` takes ``x`` as ``NormedRows`` and an ``epilogue`` for its last product
    # (see ``kernels.ops.NormedRows`` / ``AddNormEpilogue``) when ``fusable(rows)`` says so.
    supports_epilogue = False
    # True: ``forward`` takes ``residual32`` (the float32 residual stream) and may add its result to
    # it in place instead of returning it; it then returns None.
    adds_residual = False

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds()

    def fusable(self, num_rows: int) -> bool:
        return False

    def forward(self, x: torch.Tensor, inputs: "Any", cache: "Any") -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    supports_epilogue = False
    adds_residual = False            # as for mixers

    def fusable(self, num_rows: int) -> bool:
        return False

    def forward(self, x: torch.Tensor, inputs: "Any") -> torch.Tensor:
        raise NotImplementedError


class Stage(Part):
    """A step of the model outside its layers: a scale or learned positions added after the token
    table, a transform of the final hidden rows, a cap on the logits.  ``forward(x, inputs) -> x``
    (it may work in place); where it stands says what ``x`` is (``ModelSpec.after_embedding``,
    ``before_head``, ``after_head``)."""

    def forward(self, x: torch.Tensor, inputs: "Any") -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of a mixer, a feed-forward and norms around the residual stream."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: dict[str, Norm]):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = norms

    def forward(self, resid32: torch.Tensor, delta, inputs: "Any", cache: "Any",
                next_norm: "Norm | None" = None) -> tuple[torch.Tensor, Any]:
        """``delta`` is what the previous block still has to add to the residual stream, or
        ``NormedRows`` if that block already added it and prepared this block's first norm.
        ``next_norm``: the norm that will consume this block's output (the next block's first
        norm), offered so that the sum and that norm can be fused into this block's last product."""
        raise NotImplementedError

    def first_norm(self, num_rows: int) -> "Norm | None":
        """The norm this block applies first to the residual stream, if for a step of ``num_rows``
        tokens the block accepts it already applied up to the RMS factor (``NormedRows``);
        None otherwise."""
        return None


# --------------------------------------------------------------------------- registries


class Registry:
    """Name -> factory.  An unknown name is an error that lists the known ones."""

    def __init__(self, what: str):
        self.what = what
        self._items: dict[str, Callable] = {}

    def register(self, name: str, factory: Callable | None = None):
        if factory is None:
            def deco(f):
                self._items[name] = f
                return f
            return deco
        self._items[name] = factory
        return factory

    def get(self, name: str) -> Callable:
        try:
            return self._items[name]
        except KeyError:
            raise KeyError(
                f"unknown {self.what} '{name}'; known: {', '.join(sorted(self._items)) or '(none)'}"
            ) from None

    def names(self) -> list[str]:
        return sorted(self._items)

    def __contains__(self, name: str) -> bool:
        return name in self._items


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
STAGES = Registry("model stage")


def build_part(registry: Registry, spec: PartSpec, ctx: BuildContext, **extra):
    """Instantiates ``spec.kind`` from ``registry`` with the spec's parameters."""
    factory = registry.get(spec.kind)
    return factory(ctx=ctx, **spec.params, **extra)
