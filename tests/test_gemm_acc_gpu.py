"""Matmul with a seeded accumulator, ``C = C + A @ B``: the reference's general
``mma(a, b, acc)`` with ``sum0 = acc[r][c]``
(crates/sile-tile-ir/src/passes/lowering/tile_compute/mma.rs:25-260), the path its kernels take
when the accumulator does not start from ``constant(0.0)``.  The sm_100a kernels add the seed in
their epilogue; the oracle runs the per-k-tile general mma on private tiles.

Tolerances as for the plain GEMM: 1e-3 (f32) / 2e-2 (bf16, f32 accumulate) of the output scale."""
import numpy as np
import pytest

from _util import normal, rel_err, tile_mask, to_bf16_bits, uniform

pytestmark = pytest.mark.gpu
F32_TOL = 1e-3
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def sb():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import sile_b200
    return sile_b200


def _run(sb, a, b, c0, bm, bn, bk, grid=None):
    import torch
    da, db, dc = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), torch.from_numpy(c0).cuda()
    kl = sb.matmul(da, db, dc, bm, bn, bk, accumulate=True)
    if grid is not None:
        kl.grid(grid)
    kl.apply()
    sb.synchronize()
    return dc.cpu().numpy()


def test_golden_inputs_with_a_seed_through_the_exact_abi(sb):
    # the inputs of crates/sile/tests/backend_matmul.rs:29-64; every sum starts from c's value
    a = np.arange(1, 17, dtype=np.float32).reshape(4, 4)
    b = np.array([1, 0, 2, 1, 0, 1, 3, 2, 1, 0, 4, 3, 0, 1, 5, 4], np.float32).reshape(4, 4)
    seed = (100 + np.arange(16, dtype=np.float32)).reshape(4, 4)
    c = seed.copy()
    sb.bind_consts("matmul_acc", (2, 2, 2))
    sb.kernel_call("matmul_acc", [a, b, c], grid=(4, 1, 1))
    product = np.array([4, 6, 40, 30, 12, 14, 96, 70, 20, 22, 152, 110, 28, 30, 208, 150], np.float32).reshape(4, 4)
    assert np.abs(c - (seed + product)).max() < 1e-4


@pytest.mark.parametrize("kernel", ["auto", "single", "pair", "wide", "sliced"])
@pytest.mark.parametrize("m,n,k,bm,bn,bk", [
    (130, 260, 70, 2, 4, 7),      # ragged everywhere, K remainder dropped
    (384, 768, 320, 64, 64, 32),  # whole CTA tiles: the vector store path
    (700, 1100, 328, 4, 4, 8),
])
def test_f32_against_the_oracle(sb, oracle, monkeypatch, kernel, m, n, k, bm, bn, bk):
    if kernel != "auto":
        monkeypatch.setenv("SILE_CUDA_GEMM_KERNEL", kernel)
    a, b, c0 = uniform((m, k), 40 + m), uniform((k, n), 41 + n), uniform((m, n), 42 + k) * 3
    want = oracle.matmul_acc(a, b, c0, bm, bn, bk)
    got = _run(sb, a, b, c0, bm, bn, bk)
    mv, nv = m // bm * bm, n // bn * bn
    # outside whole logical tiles nothing is written: the seed survives bit for bit
    assert (got[mv:] == c0[mv:]).all() and (got[:, nv:] == c0[:, nv:]).all()
    assert rel_err(got, want) < F32_TOL


@pytest.mark.parametrize("kernel", ["single", "wide"])
def test_short_grid_adds_only_inside_launched_tiles(sb, oracle, monkeypatch, kernel):
    monkeypatch.setenv("SILE_CUDA_GEMM_KERNEL", kernel)
    a, b, c0 = uniform((512, 192), 3), uniform((192, 640), 4), uniform((512, 640), 5)
    ntg = 37  # of 8 * 10 = 80 logical 64 x 64 tiles
    got = _run(sb, a, b, c0, 64, 64, 32, grid=(ntg, 1, 1))
    want = oracle.matmul_acc(a, b, c0, 64, 64, 32, grid=(ntg, 1, 1))
    mask = tile_mask(512, 640, 64, 64, range(ntg))
    assert (got[~mask] == c0[~mask]).all()
    assert rel_err(got, want) < F32_TOL


@pytest.mark.parametrize("out_bf16", [True, False])
def test_bf16_operands(sb, oracle, out_bf16):
    import torch
    m, n, k = 512, 1024, 384
    ta, a_up = to_bf16_bits(normal((m, k), 7, 1.0 / np.sqrt(k)))
    tb, b_up = to_bf16_bits(normal((k, n), 8, 1.0 / np.sqrt(k)))
    tc, c_up = to_bf16_bits(normal((m, n), 9))
    dc = tc.cuda() if out_bf16 else tc.float().cuda()
    sb.matmul(ta.cuda(), tb.t().contiguous().cuda(), dc, 1, 1, 1, b_layout=sb._lib.LAYOUT_COL_MAJOR, accumulate=True).apply()
    sb.synchronize()
    want = oracle.matmul_acc(a_up, b_up, c_up, 1, 1, 1)
    assert rel_err(dc.float().cpu().numpy(), want) < (BF16_TOL if out_bf16 else 1e-5)
    del torch
