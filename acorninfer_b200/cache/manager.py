"""The cache manager: keys and values in pages with a block table per request, per-request
state of fixed size in slots, and the bookkeeping of who holds what.

Layers are sorted into *groups* by what they need (``KVNeeds.group_key``: head count,
head size, all keys or a window of them).  A group has a page pool of its own and one
storage tensor ``[layers_in_group, 2, num_pages, kv_heads, page_size, head_dim]``: a page
id names the same page in every layer of its group.  A request has one block table per
group; the token at position p lives in ``table[p // page_size - page_base]``, slot
``p % page_size``.  ``page_base`` counts pages given back at the front of a windowed
group's table once every later query is past them.

Life of a request: ``open`` (a state slot, zeroed), then per step ``extend`` (pages for
the step's tokens, all groups or nothing, before anything is launched), ``commit`` (the
new length; windowed groups give pages back), finally ``close`` (everything back).

Reference: ``PagedKVCache``/``PagedCacheView`` in ``acorninfer/cache/pager.py:58-259``
(one group, no window, no state slots; allocation before any write ``:172``).
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import KVNeeds, StateNeeds
from .pools import IdPool, PoolExhausted


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class CacheGroup:
    index: int
    needs: KVNeeds
    entries: list[int]                  # schedule entries whose cache lives here, in order
    pool: IdPool
    storage: object = None              # torch tensor [len(entries), 2, pages, nkv, P, d] or None

    @property
    def window(self) -> int | None:
        return self.needs.window


@dataclass(eq=False)
class RequestCache:
    """What one live request holds (compared by identity)."""

    request_id: object
    slot: int
    length: int = 0                                         # tokens committed
    tables: list[list[int]] = field(default_factory=list)   # per group: physical page ids
    page_base: list[int] = field(default_factory=list)      # per group: logical index of tables[g][0]
    closed: bool = False
    _arrays: dict = field(default_factory=dict, repr=False)  # per group: tables[g] as an int32 array, while unchanged

    def table_array(self, group: int):
        """``tables[group]`` as a numpy int32 array, rebuilt only after the table changed (a page is
        added every ``page_size`` tokens, so most steps reuse it)."""
        arr = self._arrays.get(group)
        if arr is None or arr.size != len(self.tables[group]):
            import numpy as np
            arr = np.asarray(self.tables[group], dtype=np.int32)
            self._arrays[group] = arr
        return arr


class CacheManager:
    def __init__(self, kv_needs: dict[int, KVNeeds], state_needs: dict[int, StateNeeds], num_pages,
                 page_size: int, num_slots: int, dtype=None, device=None, allocate: bool = True):
        """``kv_needs`` / ``state_needs`` map schedule-entry index -> what that entry's mixer
        keeps.  ``num_pages`` is the size of every group's pool, or a function
        ``KVNeeds -> pages`` that sizes each group's pool by what it keeps (a windowed group
        needs far fewer pages than one that keeps every key).  ``dtype`` is the element type of
        groups whose ``KVNeeds.dtype`` names none."""
        if page_size < 1 or page_size & (page_size - 1):
            raise ValueError(f"page_size must be a power of two, got {page_size}")
        self.page_size = page_size
        pages_for = num_pages if callable(num_pages) else (lambda needs: num_pages)
        self.groups: list[CacheGroup] = []
        self.entry_group: dict[int, tuple[int, int]] = {}     # entry -> (group index, layer index in group)
        by_key: dict[tuple, CacheGroup] = {}
        for entry in sorted(kv_needs):
            needs = kv_needs[entry]
            g = by_key.get(needs.group_key)
            if g is None:
                g = CacheGroup(len(self.groups), needs, [], IdPool(int(pages_for(needs)), "page"))
                by_key[needs.group_key] = g
                self.groups.append(g)
            self.entry_group[entry] = (g.index, len(g.entries))
            g.entries.append(entry)
        self.slots = IdPool(num_slots, "slot")
        self.state_needs = dict(state_needs)
        self.state: dict[int, object] = {}
        self.live: dict[object, RequestCache] = {}
        self.num_pages = max((g.pool.total for g in self.groups), default=0)
        # One page per group and one slot beyond the pools, never handed out: rows that only pad a
        # step to a captured shape write their keys, values and state there.
        self.pad_pages = [g.pool.total for g in self.groups]
        self.pad_slot = num_slots
        if allocate:
            import torch
            for g in self.groups:
                n = g.needs
                g.storage = torch.zeros((len(g.entries), 2, g.pool.total + 1, n.num_kv_heads, page_size, n.head_dim),
                                        dtype=n.dtype or dtype, device=device)
            for entry, sn in self.state_needs.items():
                self.state[entry] = torch.zeros((num_slots + 1, *sn.shape), dtype=sn.dtype or torch.float32,
                                                device=device)

    # ------------------------------------------------------------------ storage views

    def kv_pages(self, entry: int):
        """(k_pages, v_pages) of a schedule entry: each [num_pages, nkv, P, d]."""
        gi, li = self.entry_group[entry]
        st = self.groups[gi].storage
        return st[li, 0], st[li, 1]

    def group_of(self, entry: int) -> int:
        return self.entry_group[entry][0]

    def bytes_per_token(self) -> int:
        total = 0
        for g in self.groups:
            width = 2 if g.storage is None else g.storage.element_size()
            total += len(g.entries) * 2 * g.needs.num_kv_heads * g.needs.head_dim * width
        return total

    # ------------------------------------------------------------------ requests

    def open(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already open")
        (slot,) = self.slots.allocate(1)
        rc = RequestCache(request_id, slot, 0, [[] for _ in self.groups], [0 for _ in self.groups])
        self.live[request_id] = rc
        for st in self.state.values():
            st[slot].zero_()
        return rc

    def _first_needed_page(self, g: CacheGroup, length: int) -> int:
        """Logical index of the first page a query at position >= ``length`` can still read."""
        if g.window is None:
            return 0
        return max(0, (length - g.window + 1) // self.page_size)

    def pages_needed(self, rc: RequestCache | None, new_length: int) -> list[int]:
        """Per group, the pages to add so that a step can bring the request to ``new_length``."""
        want = -(-new_length // self.page_size)
        if rc is None:
            return [want] * len(self.groups)
        return [max(0, want - b - len(t)) for b, t in zip(rc.page_base, rc.tables)]

    def peak_pages(self, total_length: int, max_portion: int | None) -> list[int]:
        """Per group, the most pages a request of ``total_length`` tokens holds at once when it is
        fed in portions of at most ``max_portion`` tokens (None: in one piece)."""
        out = []
        for g in self.groups:
            full = ceil_div(total_length, self.page_size)
            if g.window is None:
                out.append(full)
            else:
                portion = total_length if max_portion is None else min(max_portion, total_length)
                out.append(min(full, ceil_div(g.window + portion, self.page_size) + 1))
        return out

    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.groups]

    def total_pages(self) -> list[int]:
        return [g.pool.total for g in self.groups]

    def can_extend(self, rc: RequestCache | None, new_length: int) -> bool:
        return all(n <= f for n, f in zip(self.pages_needed(rc, new_length), self.free_pages()))

    def extend(self, rc: RequestCache, new_length: int) -> None:
        """Takes the pages a step to ``new_length`` writes: in every group, or in none."""
        if rc.closed:
            raise ValueError(f"request {rc.request_id!r} is closed")
        if new_length < rc.length:
            raise ValueError(f"cannot extend request {rc.request_id!r} from {rc.length} to {new_length}")
        need = self.pages_needed(rc, new_length)
        if not any(need):
            return
        for g, n in zip(self.groups, need):
            if n > g.pool.num_free:
                raise PoolExhausted(
                    f"request {rc.request_id!r}: group {g.index} needs {n} page(s) for length {new_length}, "
                    f"{g.pool.num_free} free of {g.pool.total}")
        for g, n in zip(self.groups, need):
            if n:
                rc.tables[g.index].extend(g.pool.allocate(n))
                rc._arrays.pop(g.index, None)

    def trim(self, rc: RequestCache) -> None:
        """Gives back the pages taken by ``extend`` beyond the committed length: for a step that
        reserved its pages and then could not be launched."""
        keep_to = ceil_div(rc.length, self.page_size)
        for g in self.groups:
            table = rc.tables[g.index]
            keep = max(0, keep_to - rc.page_base[g.index])
            if len(table) > keep:
                g.pool.free(table[keep:])
                del table[keep:]
                rc._arrays.pop(g.index, None)

    def commit(self, rc: RequestCache, new_length: int) -> None:
        """Records that the step wrote up to ``new_length``; windowed groups give back the pages
        that no later query reads."""
        if new_length < rc.length:
            raise ValueError(f"length of request {rc.request_id!r} cannot shrink ({rc.length} -> {new_length})")
        for g in self.groups:
            if rc.page_base[g.index] + len(rc.tables[g.index]) < ceil_div(new_length, self.page_size):
                raise ValueError(f"request {rc.request_id!r}: commit to {new_length} beyond its pages")
        rc.length = new_length
        for g in self.groups:
            first = self._first_needed_page(g, new_length)
            drop = first - rc.page_base[g.index]
            if drop > 0:
                table = rc.tables[g.index]
                drop = min(drop, len(table))
                g.pool.free(table[:drop])
                del table[:drop]
                rc.page_base[g.index] += drop
                rc._arrays.pop(g.index, None)

    def close(self, rc: RequestCache) -> None:
        if rc.closed:
            raise ValueError(f"request {rc.request_id!r} closed twice")
        for g in self.groups:
            g.pool.free(rc.tables[g.index])
            rc.tables[g.index] = []
        rc._arrays.clear()
        self.slots.free([rc.slot])
        rc.closed = True
        rc.length = 0
        del self.live[rc.request_id]

    def assert_balanced(self) -> None:
        for g in self.groups:
            g.pool.assert_balanced()
        self.slots.assert_balanced()
        if self.live:
            raise RuntimeError(f"requests still open: {list(self.live)[:8]}")
