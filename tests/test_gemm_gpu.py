"""GEMM parity: the sm_100a kernel, called through the C ABI, against the CPU oracle.

Tolerances (relative to output scale max|oracle|): 1e-3 for f32, 2e-2 for bf16 with
f32 accumulation."""
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


def _gpu_matmul_f32(sb, a, b, bm, bn, bk, grid=None, c_init=None):
    import torch
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    m, n = a.shape[0], b.shape[1]
    dc = torch.zeros(m, n, device="cuda") if c_init is None else torch.from_numpy(c_init).cuda()
    kl = sb.matmul(da, db, dc, bm, bn, bk)
    if grid is not None:
        kl.grid(grid)
    kl.apply()
    sb.synchronize()
    return dc.cpu().numpy()


def test_reference_golden_4x4_exact_abi(sb):
    # crates/sile/tests/backend_matmul.rs:29-64: host buffers, tiles 2x2x2, grid (4,1,1)
    a = np.arange(1, 17, dtype=np.float32).reshape(4, 4)
    b = np.array([1, 0, 2, 1, 0, 1, 3, 2, 1, 0, 4, 3, 0, 1, 5, 4], np.float32).reshape(4, 4)
    c = np.zeros((4, 4), np.float32)
    sb.bind_consts("matmul", (2, 2, 2))
    sb.kernel_call("matmul", [a, b, c], grid=(4, 1, 1))
    expected = np.array([4, 6, 40, 30, 12, 14, 96, 70, 20, 22, 152, 110, 28, 30, 208, 150], np.float32)
    assert np.abs(c.ravel() - expected).max() < 1e-4


def test_g1_f32_512_full(sb, oracle):
    a, b = uniform((512, 512), 0), uniform((512, 512), 1)
    want = oracle.matmul(a, b, 64, 64, 32)
    got = _gpu_matmul_f32(sb, a, b, 64, 64, 32, grid=(8, 8, 1))
    assert rel_err(got, want) < F32_TOL


def test_g1_through_exact_abi(sb, oracle):
    a, b = uniform((512, 512), 0), uniform((512, 512), 1)
    c = np.zeros((512, 512), np.float32)
    sb.bind_consts("matmul", (64, 64, 32))
    sb.kernel_call("matmul", [a, b, c], grid=(8, 8, 1))
    assert rel_err(c, oracle.matmul(a, b, 64, 64, 32)) < F32_TOL


@pytest.mark.parametrize("m,n,k,bm,bn,bk", [
    (4, 4, 4, 2, 2, 2),          # one CTA tile, mostly padding
    (128, 256, 64, 32, 16, 8),   # exactly one CTA tile, one k block
    (130, 260, 70, 2, 4, 7),     # ragged everywhere, K remainder dropped (70 = 10 * 7)
    (300, 200, 100, 4, 8, 3),    # K remainder 1 dropped; odd leading dimensions
    (128, 128, 64, 32, 16, 8),   # the reference example's shape (examples/matmul.rs:24-37)
    (384, 768, 320, 64, 64, 32), # several tiles per CTA column, 5 k blocks
    (1000, 1000, 1000, 8, 8, 8),
])
def test_f32_shapes(sb, oracle, m, n, k, bm, bn, bk):
    a, b = uniform((m, k), 10 + m), uniform((k, n), 11 + n)
    sentinel = np.full((m, n), -7.0, np.float32)
    want = sentinel.copy()
    covered = oracle.matmul(a, b, bm, bn, bk)
    mv, nv = m // bm * bm, n // bn * bn
    want[:mv, :nv] = covered[:mv, :nv]
    got = _gpu_matmul_f32(sb, a, b, bm, bn, bk, c_init=sentinel)
    # rows/columns outside whole logical tiles stay untouched, exactly
    assert (got[mv:] == -7.0).all() and (got[:, nv:] == -7.0).all()
    assert rel_err(got[:mv, :nv], want[:mv, :nv]) < F32_TOL


def test_short_grid_leaves_tiles_untouched(sb, oracle):
    # cpu/codegen.rs:517-533: pids >= grid product never run
    a, b = uniform((256, 192), 3), uniform((192, 320), 4)
    sentinel = np.full((256, 320), 5.0, np.float32)
    ntg = 13  # of 4 * 5 = 20 logical tiles of 64 x 64
    got = _gpu_matmul_f32(sb, a, b, 64, 64, 32, grid=(ntg, 1, 1), c_init=sentinel)
    want = oracle.matmul(a, b, 64, 64, 32)
    mask = tile_mask(256, 320, 64, 64, range(ntg))
    assert (got[~mask] == 5.0).all()
    assert rel_err(got[mask], want[mask]) < F32_TOL


def test_zero_and_identity(sb):
    import torch
    a = uniform((256, 128), 5)
    eye = np.eye(128, dtype=np.float32)
    got = _gpu_matmul_f32(sb, a, eye, 1, 1, 1)
    assert np.abs(got - a).max() < 1e-5  # hi+lo bf16 split keeps ~17 mantissa bits
    got = _gpu_matmul_f32(sb, np.zeros_like(a), eye, 1, 1, 1)
    assert (got == 0).all()
    del torch


def _bf16_case(sb, oracle, m, n, k, b_layout_col, out_bf16=True, seed=0):
    import torch
    a32 = normal((m, k), seed, 1.0 / np.sqrt(k))
    b32 = normal((k, n), seed + 1, 1.0 / np.sqrt(k))
    ta, a_up = to_bf16_bits(a32)
    tb, b_up = to_bf16_bits(b32)
    da = ta.cuda()
    if b_layout_col:
        db = tb.t().contiguous().cuda()  # [N, K] row-major == column-major [K, N]
        layout = sb._lib.LAYOUT_COL_MAJOR
    else:
        db = tb.cuda()
        layout = sb._lib.LAYOUT_ROW_MAJOR
    dc = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16 if out_bf16 else torch.float32)
    sb.matmul(da, db, dc, 1, 1, 1, b_layout=layout).apply()
    sb.synchronize()
    return dc.float().cpu().numpy(), a_up, b_up


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (512, 768, 256), (200, 136, 72), (1024, 1024, 1024)])
@pytest.mark.parametrize("col_major", [True, False])
def test_bf16_shapes(sb, oracle, m, n, k, col_major):
    got, a_up, b_up = _bf16_case(sb, oracle, m, n, k, col_major)
    want = oracle.matmul(a_up, b_up, 1, 1, 1)
    assert rel_err(got, want) < BF16_TOL


@pytest.mark.parametrize("kernel", ["single", "pair", "wide", "sliced"])
def test_every_kernel_variant(sb, oracle, kernel, monkeypatch):
    """The single-CTA, CTA-pair (256x256), wide CTA-pair (256x512) and sliced CTA-pair (256x256
    tiles cut into column slices, TMA-store epilogue) kernels on the same problems: ragged f32
    with a K remainder and a short grid, and bf16 with several tiles."""
    monkeypatch.setenv("SILE_CUDA_GEMM_KERNEL", kernel)
    m, n, k, bm, bn, bk = 700, 1100, 328, 4, 4, 8
    a, b = uniform((m, k), 31), uniform((k, n), 32)
    sentinel = np.full((m, n), -7.0, np.float32)
    ntg = (m // bm) * (n // bn) - 37
    got = _gpu_matmul_f32(sb, a, b, bm, bn, bk, grid=(ntg, 1, 1), c_init=sentinel)
    want = oracle.matmul(a, b, bm, bn, bk)
    mask = tile_mask(m, n, bm, bn, range(ntg))
    assert (got[~mask] == -7.0).all()
    assert rel_err(got[mask], want[mask]) < F32_TOL
    got, a_up, b_up = _bf16_case(sb, oracle, 1024, 1536, 512, True, seed=5)
    assert rel_err(got, oracle.matmul(a_up, b_up, 1, 1, 1)) < BF16_TOL


def test_bf16_f32_out_is_tight(sb, oracle):
    # with f32 output only accumulation order differs from the oracle
    got, a_up, b_up = _bf16_case(sb, oracle, 256, 512, 512, True, out_bf16=False)
    assert rel_err(got, oracle.matmul(a_up, b_up, 1, 1, 1)) < 1e-5


def test_bf16_rejects_unaligned_k(sb):
    import torch
    a = torch.zeros(64, 20, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(64, 20, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(sb.SileError) as e:
        sb.matmul(a, b, c, b_layout=sb._lib.LAYOUT_COL_MAJOR).apply()
    assert e.value.code == sb._lib.ERR_UNSUPPORTED


def test_g2_f32_4096_sampled_tiles(sb, oracle):
    n = 4096
    a, b = uniform((n, n), 0), uniform((n, n), 1)
    got = _gpu_matmul_f32(sb, a, b, 64, 64, 32)
    ids = np.random.default_rng(0).choice((n // 64) ** 2, size=48, replace=False)
    want = oracle.matmul_tiles(a, b, 64, 64, 32, ids)
    mask = tile_mask(n, n, 64, 64, ids)
    scale = np.abs(want[mask]).max()
    assert rel_err(got[mask], want[mask], scale) < F32_TOL
    # size-independent property at full size: row sums of C equal A @ (B @ 1)
    ones = b.astype(np.float64).sum(axis=1)
    rows = a.astype(np.float64) @ ones
    assert np.abs(got.astype(np.float64).sum(axis=1) - rows).max() / np.abs(rows).max() < 1e-4


def test_g3_bf16_8192_sampled_tiles_and_linearity(sb, oracle):
    import torch
    n = 8192
    a32 = normal((n, n), 0, 1.0 / np.sqrt(n))
    b32 = normal((n, n), 1, 1.0 / np.sqrt(n))
    ta, a_up = to_bf16_bits(a32)
    tb, b_up = to_bf16_bits(b32)  # logical [K, N]
    da = ta.cuda()
    db = tb.t().contiguous().cuda()
    dc = torch.zeros(n, n, device="cuda", dtype=torch.bfloat16)
    sb.matmul(da, db, dc, 64, 64, 32, b_layout=sb._lib.LAYOUT_COL_MAJOR).apply()
    sb.synchronize()
    got = dc.float().cpu().numpy()
    ids = np.random.default_rng(0).choice((n // 64) ** 2, size=32, replace=False)
    want = oracle.matmul_tiles(a_up, b_up, 64, 64, 32, ids)
    mask = tile_mask(n, n, 64, 64, ids)
    assert rel_err(got[mask], want[mask], np.abs(want[mask]).max()) < BF16_TOL
    # linearity at full size: (2A) B == 2 (A B) exactly in bf16 (power-of-two scaling)
    dc2 = torch.zeros_like(dc)
    sb.matmul((da * 2).contiguous(), db, dc2, 64, 64, 32, b_layout=sb._lib.LAYOUT_COL_MAJOR).apply()
    sb.synchronize()
    assert torch.equal(dc2, dc * 2)


@pytest.mark.parametrize("ag_kernel", ["pair", "pair:off", "pair:1,1,0,2,2", "pair:2,1,1,1,0", "pair:0,0,1,-1,2", "pair:1,1,0,1,1,1,0", "wide"])
@pytest.mark.parametrize("world,m", [(2, 512), (4, 512), (8, 1000)])
def test_fused_allgather_epilogue_on_one_gpu(sb, oracle, monkeypatch, world, m, ag_kernel):
    """The GEMM whose epilogue stores its column block into every rank's buffer, with the ranks
    played one after another on a single GPU (no kernel waits on another): afterwards every
    buffer holds the whole product.  Both kernels that carry the fused epilogue -- the 256 x 256
    pair kernel (the default) and the wide one -- and a row count that leaves a ragged last tile
    (per-thread stores to every destination).  The pair kernel cuts tiles into column slices;
    the suffix names the cut: the default plan, none, or `s0,n0,s1,n1,s2` = the first n0 tiles in
    2^s0 slices, the next n1 in 2^s1, ..., the others in 2^s_last."""
    import torch
    ag_kernel, _, split = ag_kernel.partition(":")
    if split:
        monkeypatch.setenv("SILE_CUDA_GEMM_AG_SPLIT", split)
    monkeypatch.setenv("SILE_CUDA_GEMM_AG_KERNEL", ag_kernel)
    n, k = 2048, 256
    a32 = normal((m, k), 40, 1.0 / np.sqrt(k))
    b32 = normal((k, n), 41, 1.0 / np.sqrt(k))
    ta, a_up = to_bf16_bits(a32)
    tb, b_up = to_bf16_bits(b32)
    da = ta.cuda()
    db = tb.t().contiguous().cuda()          # [N, K]
    bufs = [torch.full((m, n), 9.0, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    ptrs = [b.data_ptr() for b in bufs]
    w = n // world
    for rank in range(world):
        sb.matmul_allgather(da, db[rank * w:(rank + 1) * w].contiguous(), ptrs, rank, n, torch.bfloat16)
    chosen = sb._lib.lib().sile_cuda_last_kernel().decode()
    assert chosen.startswith("gemm_tn_pair_sliced_kernel" if ag_kernel == "pair" else "gemm_tn_pair_wide_kernel"), chosen
    sb.synchronize()
    want = oracle.matmul(a_up, b_up, 1, 1, 1)
    for b in bufs:
        assert rel_err(b.float().cpu().numpy(), want) < BF16_TOL
    assert all(torch.equal(bufs[0], b) for b in bufs[1:])
    single = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    sb.matmul(da, db, single, 1, 1, 1, b_layout=sb._lib.LAYOUT_COL_MAJOR).apply()
    sb.synchronize()
    assert torch.equal(single, bufs[0])      # sharding changes nothing, bit for bit


@pytest.mark.parametrize("ag_kernel", ["pair", "wide"])
def test_fused_allgather_epilogue_with_f32_outputs(sb, oracle, monkeypatch, ag_kernel):
    """The same with f32 destinations (a 128-byte store box is 32 columns wide instead of 64)."""
    import torch
    monkeypatch.setenv("SILE_CUDA_GEMM_AG_KERNEL", ag_kernel)
    world, m, n, k = 2, 768, 1536, 192
    ta, a_up = to_bf16_bits(normal((m, k), 50, 1.0 / np.sqrt(k)))
    tb, b_up = to_bf16_bits(normal((k, n), 51, 1.0 / np.sqrt(k)))
    da, db = ta.cuda(), tb.t().contiguous().cuda()
    bufs = [torch.full((m, n), 9.0, device="cuda", dtype=torch.float32) for _ in range(world)]
    w = n // world
    for rank in range(world):
        sb.matmul_allgather(da, db[rank * w:(rank + 1) * w].contiguous(), [b.data_ptr() for b in bufs], rank, n, torch.float32)
    chosen = sb._lib.lib().sile_cuda_last_kernel().decode()
    assert chosen.startswith("gemm_tn_pair_sliced_kernel<float>" if ag_kernel == "pair" else "gemm_tn_pair_wide_kernel"), chosen
    sb.synchronize()
    assert rel_err(bufs[0].cpu().numpy(), oracle.matmul(a_up, b_up, 1, 1, 1)) < 1e-5
    assert torch.equal(bufs[0], bufs[1])


def test_sharded_entry_points_refuse_a_seeded_accumulator(sb):
    import ctypes as C
    import torch
    L = sb._lib
    a = torch.zeros(256, 64, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(512, 64, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(256, 512, device="cuda", dtype=torch.bfloat16)
    desc = sb.make_desc(L.OP_MATMUL, L.DTYPE_BF16, L.DTYPE_BF16, L.LAYOUT_COL_MAJOR, consts=(1, 1, 1), flags=L.FLAG_ACCUMULATE)
    ptrs = (C.c_void_p * 1)(c.data_ptr())
    assert L.lib().sile_cuda_matmul_allgather(C.byref(desc), a.data_ptr(), b.data_ptr(), ptrs, 1, 0, 256, 512, 64, None) == L.ERR_UNSUPPORTED
    assert L.lib().sile_cuda_matmul_shard(C.byref(desc), a.data_ptr(), b.data_ptr(), c.data_ptr(), 256, 512, 64, 0, 512, None) == L.ERR_UNSUPPORTED
    assert (c == 0).all()


@pytest.mark.parametrize("m", [4096, 4160, 4608])
def test_host_buffer_launch_pipelines_large_bf16_and_matches_device_launch(sb, m):
    """sile_cuda_launch_host streams a large 16-bit matmul in row chunks (copy in / compute /
    copy out overlapped; full 1024-row chunks, then a tapered tail: 512 + 256 + 256 rows, a
    64-row remainder, or 256 + 256); the result must equal the device-resident launch bit for bit."""
    import torch
    n, k = 4096, 8192
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.bfloat16).pin_memory()
    b = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16).pin_memory()  # [N, K]: column-major B
    c_host = torch.zeros(m, n, dtype=torch.bfloat16).pin_memory()

    class _KN:
        shape = (k, n)

        @staticmethod
        def data_ptr():
            return b.data_ptr()

    desc = sb.make_desc(sb._lib.OP_MATMUL, sb._lib.DTYPE_BF16, sb._lib.DTYPE_BF16, sb._lib.LAYOUT_COL_MAJOR, consts=(64, 64, 32))
    sb.KernelLauncher(desc, [a, _KN, c_host]).grid((m // 64, n // 64, 1)).apply_host()
    c_dev = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    sb.matmul(a.cuda(), b.cuda(), c_dev, 64, 64, 32, b_layout=sb._lib.LAYOUT_COL_MAJOR).apply()
    sb.synchronize()
    assert torch.equal(c_host, c_dev.cpu())
    ref = a[:256].float() @ b.float().t()
    assert rel_err(c_host[:256].float().numpy(), ref.numpy()) < BF16_TOL


@pytest.mark.parametrize("kernel", ["single", "wide", "sliced"])
def test_f16_inputs_and_outputs(sb, kernel, monkeypatch):
    """fp16 operands (kind::f16 with the f16 input format) and fp16 / f32 outputs."""
    import torch
    monkeypatch.setenv("SILE_CUDA_GEMM_KERNEL", kernel)
    m, n, k = 512, 1024, 384
    g = torch.Generator().manual_seed(9)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.float16)
    b = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.float16)      # [N, K]
    want = (a.double() @ b.double().t()).numpy()
    for out_dtype, tol in ((torch.float16, 2e-3), (torch.float32, 1e-5)):
        c = torch.zeros(m, n, device="cuda", dtype=out_dtype)
        sb.matmul(a.cuda(), b.cuda(), c, 1, 1, 1, b_layout=sb._lib.LAYOUT_COL_MAJOR).apply()
        sb.synchronize()
        assert rel_err(c.double().cpu().numpy(), want) < tol
