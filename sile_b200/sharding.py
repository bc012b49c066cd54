"""Host-side partitioning for the multi-GPU path (one process per GPU).

The reference is single-device (crates/sile-core/src/stream.rs:4-19); these helpers define how
the two shardable workloads split and how the pieces are laid back together:

* matmul: contiguous output-column blocks (a block of a column-major B is contiguous), the
  packed [M, N/p] results all-gathered rank-major as [p, rows, N/p] and re-laid as [rows, N];
* attention: contiguous slabs of the flattened batch*heads axis; the rank-major all-gather of
  the output slabs already is the final [BH, S, D] layout.

Everything here is pure index arithmetic so it can be exercised with CPU ranks (gloo)."""
from __future__ import annotations

from typing import List, Tuple


def column_block(n: int, world: int, rank: int) -> Tuple[int, int]:
    """(first column, column count) of ``rank``'s block; blocks are equal, n % world == 0."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n % world != 0:
        raise ValueError(f"N = {n} does not split into {world} equal column blocks")
    w = n // world
    return rank * w, w


def head_slab(bh: int, world: int, rank: int) -> Tuple[int, int]:
    """(first index, count) of ``rank``'s slab of the flattened batch*heads axis."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if bh % world != 0:
        raise ValueError(f"batch*heads = {bh} does not split into {world} equal slabs")
    w = bh // world
    return rank * w, w


def row_chunks(m: int, chunks: int) -> List[Tuple[int, int]]:
    """Splits M rows into ``chunks`` contiguous (first row, count) pieces, used to overlap the
    all-gather of chunk i with the compute of chunk i+1.  Pieces are multiples of 256 rows (the
    CTA-pair tile) except possibly the last."""
    chunks = max(1, min(chunks, (m + 255) // 256))
    per = -(-m // chunks)
    per = -(-per // 256) * 256
    out, r = [], 0
    while r < m:
        c = min(per, m - r)
        out.append((r, c))
        r += c
    return out


def unshard_columns_index(parts: int, rows: int, cols: int, j: int, r: int, c: int) -> int:
    """Flat index in the row-major [rows, parts*cols] result of element (r, c) of rank j's
    packed [rows, cols] block -- the mapping sile_cuda_unshard_columns implements."""
    return r * parts * cols + j * cols + c
