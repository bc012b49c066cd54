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


def row_slab(m: int, world: int, rank: int) -> Tuple[int, int]:
    """(first row, row count) of the slab of A that ``rank`` stages from host memory."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if m % world != 0:
        raise ValueError(f"M = {m} does not split into {world} equal row slabs")
    w = m // world
    return rank * w, w


class HostShardedMatmul:
    """The column-block matmul from HOST buffers on ``world`` ranks.

    Every rank needs all of A.  Staging all of it on every rank sends ``world`` copies of A over
    host links the GPUs share; here each rank copies only its row slab of A (and its column block
    of B) from host memory, the slabs are all-gathered device to device, the rank computes
    ``C[:, block] = A @ B[:, block]`` and copies its block back.  Host traffic per rank drops from
    ``M*K + K*N/p`` to ``(M*K + K*N)/p`` elements.  Device buffers are allocated once.

    The compute step and the tensor factory are injected so that the staging / gather / copy-back
    logic runs unchanged with CPU ranks (gloo) in the tests:
    ``compute(a_full, b_shard, c_shard)`` fills ``c_shard`` ([M, N/p]);
    ``device_empty(shape, like)`` allocates a device tensor."""

    def __init__(self, m, n, k, world, rank, dtype, compute, device_empty, all_gather):
        self.m, self.n, self.k, self.world, self.rank = m, n, k, world, rank
        self.r0, self.rows = row_slab(m, world, rank)
        self.n0, self.cols = column_block(n, world, rank)
        self.compute, self.all_gather = compute, all_gather
        self.a_full = device_empty((m, k), dtype)
        self.b_shard = device_empty((self.cols, k), dtype)   # column-major B: a block is [N/p, K]
        self.c_shard = device_empty((m, self.cols), dtype)
        self.h2d_bytes = (self.rows * k + self.cols * k) * self.a_full.element_size()
        self.d2h_bytes = m * self.cols * self.c_shard.element_size()

    def step(self, a_host, b_shard_host, c_shard_host):
        """a_host: the whole [M, K] host matrix (only this rank's slab is read);
        b_shard_host: [N/p, K]; c_shard_host: [M, N/p], written."""
        slab = self.a_full[self.r0:self.r0 + self.rows]
        slab.copy_(a_host[self.r0:self.r0 + self.rows], non_blocking=True)
        self.b_shard.copy_(b_shard_host, non_blocking=True)
        self.all_gather(self.a_full, slab)          # in place: the slab already sits at its offset
        self.compute(self.a_full, self.b_shard, self.c_shard)
        c_shard_host.copy_(self.c_shard, non_blocking=True)


def unshard_columns_index(parts: int, rows: int, cols: int, j: int, r: int, c: int) -> int:
    """Flat index in the row-major [rows, parts*cols] result of element (r, c) of rank j's
    packed [rows, cols] block -- the mapping sile_cuda_unshard_columns implements."""
    return r * parts * cols + j * cols + c
