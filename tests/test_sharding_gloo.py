"""The multi-GPU partitioning exercised with CPU ranks: two gloo processes split a matmul by
column block and an attention-shaped tensor by batch*heads, all-gather, re-lay and compare with
the unsharded result.  The per-rank compute is a numpy stand-in: what is under test is the
partition / all-gather / unshard layout that bench.py drives on GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sile_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 512, 384, 96
        rng = np.random.default_rng(0)          # same seed on every rank: same A and B
        a = rng.standard_normal((m, k)).astype(np.float32)
        b_colmajor = rng.standard_normal((n, k)).astype(np.float32)   # [N, K] = column-major B
        n0, nc = sharding.column_block(n, world, rank)
        b_shard = b_colmajor[n0:n0 + nc]                               # contiguous block
        c = np.zeros((m, n), np.float32)
        for r0, rc in sharding.row_chunks(m, 2):
            cs = a[r0:r0 + rc] @ b_shard.T                             # packed [rows, N/p]
            gathered = torch.empty(world * rc, nc)   # rank-major concatenation = [world, rc, nc]
            dist.all_gather_into_tensor(gathered, torch.from_numpy(np.ascontiguousarray(cs)))
            g = gathered.numpy().reshape(world, rc, nc)
            flat = c[r0:r0 + rc].reshape(-1)
            for j in range(world):
                idx = sharding.unshard_columns_index(world, rc, nc, j, np.arange(rc)[:, None], np.arange(nc)[None, :])
                flat[idx.reshape(-1)] = g[j].reshape(-1)
        ok_mm = np.allclose(c, a @ b_colmajor.T, atol=1e-4)

        # host-buffer path: each rank stages its row slab of A only, the slabs are all-gathered
        hm = sharding.HostShardedMatmul(
            m, n, k, world, rank, torch.float32,
            compute=lambda af, bs, cs: cs.copy_(af @ bs.T),
            device_empty=lambda shape, dt: torch.full(shape, float("nan"), dtype=dt),
            all_gather=lambda full, part: dist.all_gather_into_tensor(full, part.clone()))
        a_host = torch.from_numpy(a).clone()
        a_host[:hm.r0] = float("nan")            # rows of other ranks' slabs must never be read here
        a_host[hm.r0 + hm.rows:] = float("nan")
        c_host = torch.zeros(m, nc)
        hm.step(a_host, torch.from_numpy(np.ascontiguousarray(b_shard)), c_host)
        ok_mm = ok_mm and np.allclose(c_host.numpy(), a @ b_shard.T, atol=1e-4)
        ok_mm = ok_mm and hm.h2d_bytes == (m // world * k + nc * k) * 4

        bh, s, d = 6, 8, 4
        o_full = rng.standard_normal((bh, s, d)).astype(np.float32)    # stands for the attention output
        h0, hc = sharding.head_slab(bh, world, rank)
        out = torch.empty(bh, s, d)
        dist.all_gather_into_tensor(out, torch.from_numpy(np.ascontiguousarray(o_full[h0:h0 + hc])))
        ok_attn = np.array_equal(out.numpy(), o_full)                  # rank-major gather == final layout
        q.put((rank, bool(ok_mm), bool(ok_attn)))
    except Exception as e:  # report instead of leaving the parent waiting
        q.put((rank, False, repr(e)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_cpu_ranks_partition_gather_unshard():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=100) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] is True and r[2] is True for r in results), results


def test_partition_arithmetic():
    assert sharding.column_block(8192, 8, 3) == (3072, 1024)
    assert sharding.head_slab(256, 8, 7) == (224, 32)
    with pytest.raises(ValueError):
        sharding.column_block(100, 8, 0)
    with pytest.raises(ValueError):
        sharding.head_slab(10, 4, 4)
    chunks = sharding.row_chunks(8192, 4)
    assert chunks == [(0, 2048), (2048, 2048), (4096, 2048), (6144, 2048)]
    assert sum(c for _, c in sharding.row_chunks(1000, 3)) == 1000
    assert sharding.row_chunks(100, 4) == [(0, 100)]
