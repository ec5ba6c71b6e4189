"""Pools of interchangeable ids: cache pages and state slots.

A pool hands out ids from a LIFO free list (an id given back is the next one handed
out, so reuse shows at once in tests), refuses to free an id that is not live, and
can assert that nothing is live.  Allocation of several ids is all or nothing.
Reference: ``BlockAllocator`` in ``acorninfer/cache/pager.py:16-55``.
"""

from __future__ import annotations


class PoolExhausted(RuntimeError):
    """More ids were asked for than are free; nothing was taken."""


class IdPool:
    def __init__(self, total: int, what: str = "page"):
        if total < 0:
            raise ValueError(f"{what} pool size must be >= 0, got {total}")
        self.total = total
        self.what = what
        self._free = list(range(total - 1, -1, -1))   # pop() hands out 0 first
        self._live: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_live(self) -> int:
        return len(self._live)

    def allocate(self, n: int = 1) -> list[int]:
        if n < 0:
            raise ValueError(f"cannot allocate {n} {self.what}s")
        if n > len(self._free):
            raise PoolExhausted(f"{n} {self.what}(s) wanted, {len(self._free)} free of {self.total}")
        out = [self._free.pop() for _ in range(n)]
        self._live.update(out)
        return out

    def free(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if i not in self._live:
                raise ValueError(f"{self.what} {i} is not live (freed twice, or never allocated)")
        if len(set(ids)) != len(ids):
            raise ValueError(f"{self.what} ids listed twice in one free: {ids}")
        for i in ids:
            self._live.remove(i)
            self._free.append(i)

    def is_live(self, i: int) -> bool:
        return i in self._live

    def assert_balanced(self) -> None:
        """Raises (not an assert: it must survive ``python -O``) if any id is still live."""
        if self._live or len(self._free) != self.total:
            raise RuntimeError(f"{self.what} pool not balanced: {len(self._live)} live {sorted(self._live)[:16]}, "
                               f"{len(self._free)} free of {self.total}")
