"""One step's batch: what the caller gives, and the arrays the kernels read.

A step is a list of :class:`StepEntry`: a request (its :class:`RequestCache`), its next
tokens, and the places among them whose logits are wanted.  All entries of a step form
one flat token batch; an entry is a *row*.  ``plan_step`` lays the batch out as plain
integer arrays (host side, no device needed); ``StepWorkspace`` packs them into one
pinned staging block and copies it to the device in a single transfer.

Arrays (int32), T tokens, R rows, W wanted logits, per cache group g:
  token_ids[T], positions[T] (absolute index of the token in its request),
  token_row[T], row_start[R+1] (offsets into the token arrays), row_pos[R] (tokens of
  the request in the cache before this step), row_slot[R], logit_tokens[W],
  g.kv_len[R] (row_pos + the row's tokens), g.page_base[R], g.block_table[R, stride].

This layer knows nothing of any kernel's tiling.  A part whose kernels need further per-step
arrays (query tiles of an attention kernel, a scan's chunk table, expert offsets) declares them
through ``Part.step_arrays()``: a name and a builder ``StepPlan -> int32 ndarray``.  The builders
of all parts of a model are handed to ``plan_step``; their arrays travel in the same single
upload and reach the part as ``StepInputs.extra[name]`` (device) and ``StepPlan.extra[name]``
(host).  A builder must be a function of the plan alone.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from ..cache.manager import CacheManager, RequestCache


class BatchError(ValueError):
    """A step that cannot run as given; nothing was launched or allocated."""


@dataclass
class StepEntry:
    cache: RequestCache
    tokens: list[int]
    want: list[int] = field(default_factory=list)
    # A single decoded token whose id is still on the device: its index among the tokens the step
    # before sampled (``tokens`` then holds a placeholder).  See ``ModelRunner.step``.
    from_device: int | None = None


@dataclass
class GroupPlan:
    kv_len: np.ndarray
    page_base: np.ndarray
    block_table: np.ndarray     # [R, stride]
    max_kv_len: int


@dataclass
class StepPlan:
    """Host-side description of a step (numpy int32 arrays)."""

    num_tokens: int
    num_rows: int
    token_ids: np.ndarray
    positions: np.ndarray
    token_row: np.ndarray
    row_start: np.ndarray
    row_pos: np.ndarray
    row_slot: np.ndarray
    logit_tokens: np.ndarray
    groups: list[GroupPlan]
    row_lens: list[int]
    max_q_len: int
    all_decode: bool            # every row is a single token
    patch_dst: np.ndarray = None       # flat token indices whose ids come from the device ...
    patch_src: np.ndarray = None       # ... and where among the previous step's sampled tokens they are
    extra: dict = field(default_factory=dict)    # arrays the model's parts declared, by name (any shape, int32)

    @property
    def num_logits(self) -> int:
        return int(self.logit_tokens.size)


def _table_stride(pages: int) -> int:
    """Block-table row stride: a power of two >= 8, so few distinct strides occur over a run."""
    stride = 8
    while stride < pages:
        stride *= 2
    return stride


def validate_entries(entries: list[StepEntry], vocab_size: int, max_tokens: int | None = None) -> None:
    if not entries:
        raise BatchError("a step needs at least one entry")
    seen = set()
    total = 0
    for e in entries:
        rid = e.cache.request_id
        if e.cache.closed:
            raise BatchError(f"request {rid!r} is closed")
        if id(e.cache) in seen:
            raise BatchError(f"request {rid!r} appears twice in one step")
        seen.add(id(e.cache))
        if len(e.tokens) < 1:
            raise BatchError(f"request {rid!r} brings no tokens")
        if e.from_device is not None and len(e.tokens) != 1:
            raise BatchError(f"request {rid!r}: only a single decoded token can take its id from the device")
        if min(e.tokens) < 0 or max(e.tokens) >= vocab_size:
            bad = next(t for t in e.tokens if not (0 <= int(t) < vocab_size))
            raise BatchError(f"request {rid!r}: token id {bad} outside the vocabulary (0..{vocab_size - 1})")
        for w in e.want:
            if not (0 <= int(w) < len(e.tokens)):
                raise BatchError(f"request {rid!r}: wanted place {w} outside its {len(e.tokens)} tokens")
        total += len(e.tokens)
    if max_tokens is not None and total > max_tokens:
        raise BatchError(f"step has {total} tokens, the workspace holds {max_tokens}")


def build_extra(plan: StepPlan, builders: dict | None) -> dict:
    """The arrays the parts declared, built for ``plan``."""
    out = {}
    for name, build in (builders or {}).items():
        arr = np.ascontiguousarray(build(plan), dtype=np.int32)
        out[name] = arr
    return out


def plan_step(entries: list[StepEntry], manager: CacheManager, builders: dict | None = None) -> StepPlan:
    """Lays out a validated step whose pages are already reserved (``manager.extend`` done).
    ``builders``: name -> function of the plan, for the arrays the model's parts declared."""
    R = len(entries)
    lens = [len(e.tokens) for e in entries]
    T = sum(lens)
    i32 = np.int32
    starts = [e.cache.length for e in entries]
    row_pos = np.asarray(starts, i32)
    row_slot = np.asarray([e.cache.slot for e in entries], i32)
    lens_a = np.asarray(lens, i32)
    row_start = np.zeros(R + 1, i32)
    np.cumsum(lens_a, out=row_start[1:])
    token_row = np.repeat(np.arange(R, dtype=i32), lens_a)
    # position of a token = tokens of its request before the step + its index within the row
    positions = (np.arange(T, dtype=i32) - row_start[token_row] + row_pos[token_row]).astype(i32, copy=False)
    if T == R:
        token_ids = np.asarray([e.tokens[0] for e in entries], i32)
    else:
        flat: list[int] = []
        for e in entries:
            flat.extend(e.tokens)
        token_ids = np.asarray(flat, i32)
    logit_tokens = [int(row_start[r]) + int(w) for r, e in enumerate(entries) for w in e.want]
    groups = []
    P = manager.page_size
    for g in manager.groups:
        gi = g.index
        stride = _table_stride(max((len(e.cache.tables[gi]) for e in entries), default=0))
        bt = np.zeros((R, stride), i32)
        base = np.asarray([e.cache.page_base[gi] for e in entries], i32)
        kv_len = row_pos + lens_a
        for r, e in enumerate(entries):
            t = e.cache.table_array(gi)
            if (int(base[r]) + t.size) * P < int(kv_len[r]):
                raise BatchError(f"request {e.cache.request_id!r}: pages of group {gi} do not cover length {int(kv_len[r])}")
            bt[r, :t.size] = t
        groups.append(GroupPlan(kv_len, base, bt, int(kv_len.max()) if R else 0))
    patch = [(int(row_start[r]), e.from_device) for r, e in enumerate(entries) if e.from_device is not None]
    plan = StepPlan(T, R, token_ids, positions, token_row, row_start, row_pos, row_slot,
                    np.asarray(logit_tokens, np.int32), groups, lens, max(lens), all(n == 1 for n in lens),
                    np.asarray([p[0] for p in patch], np.int32), np.asarray([p[1] for p in patch], np.int32))
    plan.extra = build_extra(plan, builders)
    return plan


# Row counts that all-decode steps are padded to, so that few shapes are captured as CUDA graphs.
DECODE_BUCKETS = (1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16, 20, 24, 28, 32, 40, 48, 56, 64, 80, 96, 112, 128)


def decode_bucket(n: int) -> int:
    for b in DECODE_BUCKETS:
        if n <= b:
            return b
    return -(-n // 32) * 32


def pad_decode_plan(plan: StepPlan, pad_pages: list[int], pad_slot: int, builders: dict | None = None) -> StepPlan:
    """An all-decode plan padded to its bucket: the added rows feed token 0 at position 0 of a
    request that exists only as the manager's padding pages (one per cache group) and slot; the added wanted places point
    at them.  Callers use the first ``plan.num_rows`` / ``plan.num_logits`` results only.  The parts'
    arrays are built again for the padded plan, so their sizes follow the bucket."""
    R, W = plan.num_rows, plan.num_logits
    Rb, Wb = decode_bucket(R), decode_bucket(W) if W else 0
    if Rb == R and Wb == W:
        return plan
    extra = Rb - R
    i32 = np.int32
    cat = lambda a, fill, n: np.concatenate([a, np.full(n, fill, i32)])
    groups = []
    for g, pad_page in zip(plan.groups, pad_pages):
        bt = np.zeros((Rb, g.block_table.shape[1]), i32)
        bt[:R] = g.block_table
        bt[R:, 0] = pad_page
        groups.append(GroupPlan(cat(g.kv_len, 1, extra), cat(g.page_base, 0, extra), bt, g.max_kv_len))
    pad_target = R if extra else 0                     # a padding row if there is one, else any row
    padded = StepPlan(
        Rb, Rb, cat(plan.token_ids, 0, extra), cat(plan.positions, 0, extra),
        np.arange(Rb, dtype=i32), np.arange(Rb + 1, dtype=i32), cat(plan.row_pos, 0, extra),
        cat(plan.row_slot, pad_slot, extra), cat(plan.logit_tokens, pad_target, Wb - W), groups,
        plan.row_lens + [1] * extra, 1, True, plan.patch_dst, plan.patch_src)
    padded.extra = build_extra(padded, builders)
    return padded


# A prompt portion that is a step of its own is padded to a bucket of token counts, so that a few captured
# graphs serve every length: multiples of 32 up to 512 tokens, of 64 up to 1,024 (the padding is work: at most
# a sixteenth of the step above 512 tokens, where a replayed step is 7 to 9 % faster than one launched op by op
# even at 8B sizes; below, such steps are bound by the host that launches them).
PREFILL_BUCKET = 32
PREFILL_GRAPH_MAX_TOKENS = 1024


def prefill_bucket(n: int) -> int:
    step = PREFILL_BUCKET if n <= 512 else 2 * PREFILL_BUCKET
    return -(-n // step) * step


def prefill_buckets() -> list[int]:
    """Every bucket up to the limit."""
    out, n = [], 1
    while n <= PREFILL_GRAPH_MAX_TOKENS:
        b = prefill_bucket(n)
        out.append(b)
        n = b + 1
    return out


def pad_prefill_plan(plan: StepPlan, pad_pages: list[int], page_size: int, builders: dict | None = None) -> StepPlan:
    """A step of one row of several tokens, padded to its bucket: the added tokens (id 0) continue the
    row at the positions after its last token.  Their keys and values fall either into the slots of the
    row's last page that lie beyond its length (the request's next tokens overwrite them before anything
    reads them) or, past the pages the row holds, into the manager's padding page, which the added table
    entries name.  Causal attention keeps them out of every real token's result; callers use the logits of
    the wanted places only, which do not move.  The parts' arrays are built again for the padded plan."""
    T = plan.num_tokens
    Tb = prefill_bucket(T)
    if plan.num_rows != 1 or Tb == T:
        return plan
    extra = Tb - T
    i32 = np.int32
    start = int(plan.row_pos[0])
    groups = []
    for g, pad_page in zip(plan.groups, pad_pages):
        kv_len = (g.kv_len + extra).astype(i32)
        base = int(g.page_base[0])
        need = -(-int(kv_len[0]) // page_size) - base             # table entries the padded row reads and writes
        have = -(-(start + T) // page_size) - base                # entries that name pages the row holds
        stride = max(g.block_table.shape[1], _table_stride(need))
        bt = np.zeros((1, stride), i32)
        bt[0, :g.block_table.shape[1]] = g.block_table[0]
        bt[0, have:need] = pad_page
        groups.append(GroupPlan(kv_len, g.page_base, bt, int(kv_len[0])))
    padded = StepPlan(
        Tb, 1, np.concatenate([plan.token_ids, np.zeros(extra, i32)]),
        np.concatenate([plan.positions, np.arange(start + T, start + Tb, dtype=i32)]),
        np.zeros(Tb, i32), np.asarray([0, Tb], i32), plan.row_pos, plan.row_slot, plan.logit_tokens, groups,
        [Tb], Tb, False, plan.patch_dst, plan.patch_src)
    padded.extra = build_extra(padded, builders)
    return padded


# --------------------------------------------------------------------------- device side


@dataclass
class GroupInputs:
    kv_len: object
    page_base: object
    block_table: object         # [R, stride] view
    max_kv_len: int


@dataclass
class StepInputs:
    """Device views of a step's arrays, plus the host-side facts launches need."""

    num_tokens: int
    num_rows: int
    token_ids: object
    positions: object
    token_row: object
    row_start: object
    row_pos: object
    row_slot: object
    logit_tokens: object
    groups: list[GroupInputs]
    plan: StepPlan
    patch_dst: object = None
    patch_src: object = None
    extra: dict = field(default_factory=dict)    # device views of the arrays the parts declared, by name

    @property
    def num_logits(self) -> int:
        return self.plan.num_logits


class StepWorkspace:
    """Pinned staging blocks and a device block that a step's arrays are packed into.

    The address of every array a model reads is a function of ``shape_key(plan)``: (T, R, W,
    the groups' table strides, the sizes of the parts' arrays).  Two steps of the same key put
    those arrays at the same device addresses, so a captured CUDA graph of one can be replayed
    for the other after ``upload``.  ``patch_dst`` / ``patch_src`` (read by the patch kernel,
    which runs outside any captured graph) vary in size between steps of one key and therefore
    lie behind everything else.
    """

    def __init__(self, device, capacity_ints: int = 1 << 20, num_staging: int = 3):
        import torch
        self.torch = torch
        self.device = device
        self.capacity = capacity_ints
        self.device_block = torch.zeros(capacity_ints, dtype=torch.int32, device=device)
        self.staging = [torch.zeros(capacity_ints, dtype=torch.int32).pin_memory() for _ in range(num_staging)]
        self.events = [None] * num_staging
        self._next = 0

    @staticmethod
    def layout(plan: StepPlan) -> tuple[dict, int]:
        """Offsets (in int32 elements, 4-aligned) of every array in the block."""
        off = 0
        out = {}

        def put(name, n):
            nonlocal off
            out[name] = (off, n)
            off += (n + 3) // 4 * 4

        T, R = plan.num_tokens, plan.num_rows
        put("token_ids", T)
        put("positions", T)
        put("token_row", T)
        put("row_start", R + 1)
        put("row_pos", R)
        put("row_slot", R)
        put("logit_tokens", plan.num_logits)
        for i, g in enumerate(plan.groups):
            put(f"g{i}.kv_len", R)
            put(f"g{i}.page_base", R)
            put(f"g{i}.block_table", g.block_table.size)
        for name in sorted(plan.extra):
            put("x." + name, plan.extra[name].size)
        put("patch_dst", plan.patch_dst.size)       # last: their sizes are not part of the shape key
        put("patch_src", plan.patch_src.size)
        return out, off

    @staticmethod
    def shape_key(plan: StepPlan) -> tuple:
        """What fixes the address of every array but the patch lists (see the class docstring)."""
        return (plan.num_tokens, plan.num_rows, plan.num_logits, tuple(g.block_table.shape[1] for g in plan.groups),
                tuple((name, plan.extra[name].shape) for name in sorted(plan.extra)))

    def upload(self, plan: StepPlan) -> StepInputs:
        torch = self.torch
        lay, total = self.layout(plan)
        if total > self.capacity:
            raise BatchError(f"step arrays need {total} ints, workspace holds {self.capacity}")
        i = self._next
        self._next = (self._next + 1) % len(self.staging)
        if self.events[i] is not None:
            self.events[i].synchronize()
        host = self.staging[i].numpy()
        arrays = {
            "token_ids": plan.token_ids, "positions": plan.positions, "token_row": plan.token_row,
            "row_start": plan.row_start, "row_pos": plan.row_pos, "row_slot": plan.row_slot,
            "logit_tokens": plan.logit_tokens, "patch_dst": plan.patch_dst, "patch_src": plan.patch_src,
        }
        for name, arr in plan.extra.items():
            arrays["x." + name] = arr.reshape(-1)
        for gi, g in enumerate(plan.groups):
            arrays[f"g{gi}.kv_len"] = g.kv_len
            arrays[f"g{gi}.page_base"] = g.page_base
            arrays[f"g{gi}.block_table"] = g.block_table.reshape(-1)
        for name, arr in arrays.items():
            off, n = lay[name]
            host[off:off + n] = arr
        self.device_block[:total].copy_(self.staging[i][:total], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev

        def view(name):
            off, n = lay[name]
            return self.device_block[off:off + n]

        groups = []
        for gi, g in enumerate(plan.groups):
            bt = view(f"g{gi}.block_table").view(plan.num_rows, g.block_table.shape[1])
            groups.append(GroupInputs(view(f"g{gi}.kv_len"), view(f"g{gi}.page_base"), bt, g.max_kv_len))
        return StepInputs(plan.num_tokens, plan.num_rows, view("token_ids"), view("positions"), view("token_row"),
                          view("row_start"), view("row_pos"), view("row_slot"), view("logit_tokens"), groups, plan,
                          view("patch_dst"), view("patch_src"),
                          {name: view("x." + name).view(arr.shape) for name, arr in plan.extra.items()})
