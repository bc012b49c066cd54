"""The allocation-free f32 matmul entry point against the ordinary one.

Some hosts cannot let this library allocate device memory (their own arena owns all of HBM, or
allocation is forbidden after start-up); for them ``sile_cuda_matmul_f32_noalloc`` keeps its
scratch in a fixed 32 MiB array inside the library.  This file is named to be collected last:
a run that stops at the first failure has then already run every other test.  It passes both
alone in a fresh process (the entry point does its own per-device set-up on first use) and
after the other tests."""
import ctypes as C

import numpy as np
import pytest

from _util import rel_err, uniform

pytestmark = pytest.mark.gpu
F32_TOL = 1e-3  # max-abs error relative to output scale, as in test_gemm_gpu.py


@pytest.fixture(scope="module")
def sb():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import sile_b200
    return sile_b200


def _noalloc(sb, da, db, dc, bm, bn, bk, wait=1):
    import torch
    m, k = da.shape
    n = db.shape[1]
    rc = sb._lib.lib().sile_cuda_matmul_f32_noalloc(
        da.data_ptr(), db.data_ptr(), dc.data_ptr(), m, n, k, bm, bn, bk,
        C.c_void_p(torch.cuda.current_stream().cuda_stream), wait)
    return rc


def test_two_calls_in_a_row_match_the_allocating_entry_point(sb):
    import torch
    # second call is smaller in every dimension and has a K remainder: stale planes from the
    # first call lie right behind and inside its scratch region
    cases = [((1024, 768, 1000), (64, 64, 32)), ((300, 200, 100), (4, 8, 3))]
    for (m, n, k), (bm, bn, bk) in cases:
        a, b = uniform((m, k), 21 + m), uniform((k, n), 22 + n)
        da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        want = torch.full((m, n), -7.0, device="cuda")
        sb.matmul(da, db, want, bm, bn, bk).apply()
        sb.synchronize()
        got = torch.full((m, n), -7.0, device="cuda")
        assert _noalloc(sb, da, db, got, bm, bn, bk) == 0, sb._lib.lib().sile_cuda_last_error()
        got, want = got.cpu().numpy(), want.cpu().numpy()
        mv, nv = m // bm * bm, n // bn * bn
        assert (got[mv:] == -7.0).all() and (got[:, nv:] == -7.0).all()
        assert rel_err(got[:mv, :nv], want[:mv, :nv]) < F32_TOL
        assert rel_err(got[:mv, :nv], a[:mv, :k // bk * bk].astype(np.float64) @ b[:k // bk * bk, :nv]) < F32_TOL


def test_no_device_memory_is_allocated_and_k_below_bk(sb):
    """What the entry point exists for: after its first call on the device, further calls of any
    admissible size change neither the free memory the driver reports nor what the default
    stream-ordered pool has reserved.  One of the sizes has K < BK: no k step runs, the planes are
    all zero padding and every whole logical tile of C becomes 0.0, as with the allocating path."""
    import torch
    a, b = uniform((128, 64), 3), uniform((64, 128), 4)
    warm = torch.zeros(128, 128, device="cuda")
    assert _noalloc(sb, torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), warm, 1, 1, 1) == 0
    cases = [(640, 512, 384, (64, 64, 32)), (96, 200, 24, (32, 40, 32)), (1000, 1000, 1000, (8, 8, 8))]
    inputs = []
    for m, n, k, tile in cases:
        da, db = torch.from_numpy(uniform((m, k), m)).cuda(), torch.from_numpy(uniform((k, n), n)).cuda()
        inputs.append((da, db, torch.full((m, n), -7.0, device="cuda"), torch.full((m, n), -7.0, device="cuda"), tile))
    torch.cuda.synchronize()
    pool = torch.cuda.memory.memory_stats()  # torch's own allocator must not move either
    free_before = torch.cuda.mem_get_info()[0]
    reserved_before = torch.cuda.memory_reserved()
    for da, db, got, _, (bm, bn, bk) in inputs:
        assert _noalloc(sb, da, db, got, bm, bn, bk) == 0, sb._lib.lib().sile_cuda_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    del pool
    for da, db, got, want, (bm, bn, bk) in inputs:
        sb.matmul(da, db, want, bm, bn, bk).apply()
        sb.synchronize()
        m, n = got.shape
        mv, nv = m // bm * bm, n // bn * bn
        g, w = got.cpu().numpy(), want.cpu().numpy()
        assert (g[mv:] == -7.0).all() and (g[:, nv:] == -7.0).all()
        scale = max(np.abs(w[:mv, :nv]).max(), 1.0)
        assert np.abs(g[:mv, :nv] - w[:mv, :nv]).max() < F32_TOL * scale
    # K = 24 < BK = 32: zero k steps, whole logical tiles become exactly 0.0
    assert (inputs[1][2].cpu().numpy()[:96, :200] == 0.0).all()


def test_asynchronous_form_and_size_limit(sb):
    import torch
    a, b = uniform((256, 512), 1), uniform((512, 384), 2)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    got = torch.zeros(256, 384, device="cuda")
    assert _noalloc(sb, da, db, got, 1, 1, 1, wait=0) == 0
    torch.cuda.synchronize()
    assert rel_err(got.cpu().numpy(), a.astype(np.float64) @ b) < F32_TOL
    # 4 * (M + N) * K = 4 * 8192 * 4096 = 128 MiB > 32 MiB: rejected, nothing launched
    big_a = torch.zeros(4096, 4096, device="cuda")
    out = torch.full((4096, 4096), 5.0, device="cuda")
    rc = _noalloc(sb, big_a, big_a, out, 1, 1, 1)
    assert rc == sb._lib.ERR_UNSUPPORTED
    assert b"32" in sb._lib.lib().sile_cuda_last_error() or b"33554432" in sb._lib.lib().sile_cuda_last_error()
    assert (out == 5.0).all().item()
