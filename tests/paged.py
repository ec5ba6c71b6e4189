"""Helpers that build paged caches and step arrays by hand for kernel tests."""

from __future__ import annotations

import random

import torch


def rows_layout(kv_before: list[int], q_lens: list[int], P: int, num_pages: int, seed: int = 0, device="cuda:0"):
    """Block tables over a shuffled page pool for rows that hold ``kv_before[r]`` tokens and
    bring ``q_lens[r]`` new ones.  Returns a dict of int32 device tensors and the host tables."""
    rng = random.Random(seed)
    pool = list(range(num_pages))
    rng.shuffle(pool)
    tables = []
    for before, q in zip(kv_before, q_lens):
        n = -(-(before + q) // P)
        tables.append([pool.pop() for _ in range(n)])
    stride = max(len(t) for t in tables) + 3          # a stride that is not the table length
    bt = torch.zeros((len(tables), stride), dtype=torch.int32)
    for r, t in enumerate(tables):
        bt[r, :len(t)] = torch.tensor(t, dtype=torch.int32)
    token_row, positions = [], []
    for r, (before, q) in enumerate(zip(kv_before, q_lens)):
        token_row += [r] * q
        positions += list(range(before, before + q))
    i32 = dict(dtype=torch.int32, device=device)
    return {
        "block_table": bt.to(device), "page_base": torch.zeros(len(tables), **i32),
        "token_row": torch.tensor(token_row, **i32), "positions": torch.tensor(positions, **i32),
        "tables": tables, "num_tokens": len(token_row),
    }


def scatter_to_pages(pages: torch.Tensor, table: list[int], dense: torch.Tensor, P: int, start: int = 0):
    """pages [num_pages, nkv, P, d]; dense [S, nkv, d] holds tokens start..start+S of a row."""
    for i in range(dense.shape[0]):
        pos = start + i
        pages[table[pos // P], :, pos % P, :] = dense[i].to(pages.dtype)


def gather_from_pages(pages: torch.Tensor, table: list[int], length: int, P: int) -> torch.Tensor:
    """The first ``length`` tokens of a row as [length, nkv, d]."""
    return torch.stack([pages[table[pos // P], :, pos % P, :] for pos in range(length)])
