"""How the path is partitioned over the GPUs of one node (host-side index arithmetic only).

* Decode requests are independent: rank r owns a contiguous block of requests, weights are
  replicated, nothing is exchanged.
* The one large layer is split by output columns: rank r owns columns [n0, n1) of the
  K-major weight (`[K/32][N]` blocks), computes y[:, n0:n1] into slot r of a
  `[world][m][n/world]` gather buffer, and one all-gather completes the buffer on every rank.
"""
from __future__ import annotations

import numpy as np


def request_shard(total: int, world: int, rank: int) -> slice:
    """Requests of `rank` when `total` requests are dealt out in contiguous, near-equal blocks."""
    if world <= 0 or not (0 <= rank < world) or total < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return slice(lo, lo + base + (1 if rank < extra else 0))


def column_shard(n: int, world: int, rank: int, multiple: int = 32) -> tuple[int, int]:
    """Columns [n0, n1) of `rank`. Equal shares, each a multiple of `multiple` so that any
    `QuantBlockOrder` row group and the tiled kernels' groups of 8 columns stay whole."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad shard arguments")
    if n % (world * multiple) != 0:
        raise ValueError(f"{n} columns do not split into {world} shares that are multiples of {multiple}")
    per = n // world
    return rank * per, (rank + 1) * per


def slice_kmajor_columns(blocks: np.ndarray, kblocks: int, n: int, block_bytes: int, n0: int, n1: int) -> np.ndarray:
    """Columns [n0, n1) of a K-major `[kblocks][n]` block array, as a contiguous `[kblocks][n1 - n0]` array."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(kblocks, n, block_bytes)
    return np.ascontiguousarray(b[:, n0:n1, :]).reshape(-1)


def assemble_gathered(gather: np.ndarray) -> np.ndarray:
    """`[world][m][n_loc]` gather buffer -> y `[m][world * n_loc]`."""
    world, m, n_loc = gather.shape
    return np.ascontiguousarray(np.transpose(gather, (1, 0, 2))).reshape(m, world * n_loc)
