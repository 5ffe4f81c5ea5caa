"""CPU restatement of KV block movement (move, swap, block-table remap) in numpy.

TEST INFRASTRUCTURE ONLY: imported by ``tests/`` and by ``bench.py``'s CPU
baseline; the product path never calls it.

Parity unpinned: the reference names these operators as its next ones
(docs/operator-catalog.md:61 "KV block copy, swap, gather, scatter, compact,
and remap"; docs/operator-catalog.md:140) but has no implementation, test or
golden vector for them. The semantics restated here are the ones declared in
``include/loom_launch.h`` part 3: a cache is ``[blocks, 2, block_bytes]`` bytes
(K part and V part of every block), ids outside a cache make the pair a no-op.
"""

from __future__ import annotations

import numpy as np


def as_block_bytes(cache: np.ndarray) -> np.ndarray:
    """``[blocks, 2, ...]`` of any dtype -> ``[blocks, 2, block_bytes]`` uint8 copy (logical order)."""
    dense = np.ascontiguousarray(cache)
    return dense.view(np.uint8).reshape(dense.shape[0], 2, -1).copy()


def kv_block_move(destination: np.ndarray, source: np.ndarray, pairs: np.ndarray) -> np.ndarray:
    """destination[pairs[i, 1]] = source[pairs[i, 0]] for every pair with both ids in range."""
    out = destination.copy()
    for from_block, to_block in np.asarray(pairs, dtype=np.int64).reshape(-1, 2):
        if 0 <= from_block < source.shape[0] and 0 <= to_block < out.shape[0]:
            out[to_block] = source[from_block]
    return out


def kv_block_swap(cache: np.ndarray, pairs: np.ndarray) -> np.ndarray:
    """Exchanges blocks pairs[i, 0] and pairs[i, 1] for every pair with both ids in range."""
    out = cache.copy()
    for left, right in np.asarray(pairs, dtype=np.int64).reshape(-1, 2):
        if 0 <= left < out.shape[0] and 0 <= right < out.shape[0] and left != right:
            out[left], out[right] = cache[right], cache[left]
    return out


def block_table_remap(tables: np.ndarray, new_ids: np.ndarray) -> np.ndarray:
    """tables[i] = new_ids[tables[i]] where 0 <= tables[i] < len(new_ids); other entries stay."""
    out = tables.copy()
    inside = (tables >= 0) & (tables < new_ids.shape[0])
    out[inside] = new_ids[tables[inside]]
    return out


def compaction_plan(live: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Moves that pack the live blocks (boolean mask) to the front of the cache.

    Returns (pairs [n, 2] int64, new_ids [blocks] int32). A live block above the
    live count moves into the lowest free slot below it; blocks that stay keep
    their id. No block is both read and written.
    """
    live = np.asarray(live, dtype=bool)
    count = int(live.sum())
    holes = [b for b in range(count) if not live[b]]
    movers = [b for b in range(count, live.shape[0]) if live[b]]
    new_ids = np.arange(live.shape[0], dtype=np.int32)
    pairs = np.zeros((len(movers), 2), dtype=np.int64)
    for i, (from_block, to_block) in enumerate(zip(movers, holes)):
        pairs[i] = (from_block, to_block)
        new_ids[from_block] = to_block
    return pairs, new_ids
