"""Standalone tile ops (vec_add, relu, softmax, parallel_reduce, matvec) through the C ABI
against the reference's golden vectors and the CPU oracle."""
import numpy as np
import pytest

from _util import uniform

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sb():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import sile_b200
    return sile_b200


def test_vec_add_golden(sb):
    # crates/sile/tests/backend_vec_add.rs:15-24
    a, b, c = np.full(16, 1.0, np.float32), np.full(16, 2.0, np.float32), np.zeros(16, np.float32)
    sb.bind_consts("vec_add", (4,))
    sb.kernel_call("vec_add", [a, b, c], grid=(4, 1, 1))
    assert (c == 3.0).all()


def test_vec_add_short_grid_and_large(sb, oracle):
    a, b = uniform(1 << 20, 0), uniform(1 << 20, 1)
    c = np.full(1 << 20, 9.0, np.float32)
    want = c.copy()
    sb.bind_consts("vec_add", (4,))
    sb.kernel_call("vec_add", [a, b, c], grid=(1000, 1, 1))
    oracle.lib.sile_oracle_bind_vec_add(4)
    oracle.launch("vec_add", [a, b, want], grid=(1000, 1, 1))
    assert (c == want).all()  # bit-exact: one rounded add per element
    c2 = np.zeros(1 << 20, np.float32)
    sb.kernel_call("vec_add", [a, b, c2], grid=(1 << 18, 1, 1))
    assert (c2 == a + b).all()


def test_relu_golden(sb):
    # crates/sile/tests/llvm_ir_cpu_runtime.rs:118-140
    x = np.array([-3.0, -1.0, 0.0, 2.5, 4.0, -7.0, 8.0, -0.5], np.float32)
    sb.kernel_call("relu", [x], grid=(1, 1, 1))
    assert (x == np.array([0, 0, 0, 2.5, 4.0, 0, 8.0, 0], np.float32)).all()


def test_relu_large_matches_oracle(sb, oracle):
    x = uniform(100_003, 3)
    want = x.copy()
    oracle.launch("relu", [want])
    sb.kernel_call("relu", [x])
    assert (x == want).all()


def test_softmax_golden(sb):
    # crates/sile/tests/backend_softmax.rs:21-37
    x = np.arange(32, dtype=np.float32).reshape(4, 8)
    y = np.zeros((4, 8), np.float32)
    sb.bind_consts("softmax", (2, 8))
    sb.kernel_call("softmax", [x, y], grid=(2, 1, 1))
    assert np.abs(y.sum(axis=1) - 1.0).max() < 1e-4


# vector path (cols % 4 == 0, <= 1024; 1, 2, 4 and 8 float4 per lane, ragged last chunk), scalar
# register-cached path (odd cols), and the long-row path (> 1024)
@pytest.mark.parametrize("rows,cols", [(64, 8), (65, 36), (50, 128), (37, 260), (333, 1000), (129, 1024), (40, 1023), (16, 4096)])
def test_softmax_matches_oracle(sb, oracle, rows, cols):
    x = uniform((rows, cols), 7) * 8
    y = np.zeros_like(x)
    want = np.zeros_like(x)
    sb.bind_consts("softmax", (1, cols))
    sb.kernel_call("softmax", [x, y], grid=(rows, 1, 1))
    oracle.lib.sile_oracle_bind_softmax(1, cols)
    oracle.launch("softmax", [x, want], grid=(rows, 1, 1))
    assert np.abs(y - want).max() < 1e-3 * want.max()
    assert np.abs(y.sum(axis=1) - 1.0).max() < 1e-4


@pytest.mark.parametrize("rows,cols,bm,bn,short", [
    (4, 8, 2, 4, 0),        # the reference example's tensor with half-row tiles
    (64, 96, 8, 32, 0),
    (33, 100, 4, 24, 0),    # rows and columns past the last whole tile stay untouched
    (40, 1024, 5, 128, 7),  # a short grid stops in the middle of a tile row
    (6, 4096, 3, 2048, 1),  # tiles longer than the register-cached row kernels handle
])
def test_tile_local_softmax_matches_oracle(sb, oracle, rows, cols, bm, bn, short):
    """BN narrower than the row: every [BM, BN] tile is normalised on its own, as the reference's
    kernel does (crates/sile/examples/softmax.rs:3-16)."""
    x = uniform((rows, cols), 17) * 6
    y = np.full_like(x, -3.0)
    want = np.full_like(x, -3.0)
    ntg = (rows // bm) * (cols // bn) - short
    sb.bind_consts("softmax", (bm, bn))
    sb.kernel_call("softmax", [x, y], grid=(ntg, 1, 1))
    oracle.lib.sile_oracle_bind_softmax(bm, bn)
    oracle.launch("softmax", [x, want], grid=(ntg, 1, 1))
    untouched = want == -3.0
    assert (y[untouched] == -3.0).all()
    assert np.abs(y - want)[~untouched].max() < 1e-3 * want[~untouched].max()


def test_parallel_reduce_golden(sb):
    # crates/sile/tests/backend_parallel_reduce.rs:16-28
    a = np.ones(100_000, np.float32)
    out = np.zeros(1, np.float32)
    sb.bind_consts("parallel_reduce", (1000,))
    sb.kernel_call("parallel_reduce", [a, out], grid=(100, 1, 1))
    assert abs(out[0] - 100_000.0) < 1e-4


def test_parallel_reduce_accumulates_and_matches_oracle(sb, oracle):
    a = uniform(1 << 22, 5)
    out = np.array([3.0], np.float32)
    want = np.array([3.0], np.float32)
    sb.bind_consts("parallel_reduce", (1024,))
    sb.kernel_call("parallel_reduce", [a, out], grid=(1 << 12, 1, 1))
    oracle.lib.sile_oracle_bind_parallel_reduce(1024)
    oracle.launch("parallel_reduce", [a, want], grid=(1 << 12, 1, 1))
    # examples/parallel_reduce.rs:26-29 checks a relative 1e-5 against the exact sum
    exact = 3.0 + a.astype(np.float64).sum()
    assert abs(out[0] - exact) < 1e-3 * np.abs(a).sum() * 1e-2
    assert abs(out[0] - want[0]) < 1e-3 * np.sqrt(a.size)


def test_mlp_chain(sb, oracle):
    # crates/sile/examples/mlp.rs:60-146: gemm -> matvec -> relu, tolerance 1e-3
    rng = np.random.default_rng(2)
    w0, w1, x = rng.random((64, 64), dtype=np.float32), rng.random(64, dtype=np.float32), rng.random((64, 64), dtype=np.float32)
    out0 = np.zeros((64, 64), np.float32)
    out1 = np.zeros(64, np.float32)
    sb.bind_consts("matmul", (32, 32, 8))
    sb.kernel_call("matmul", [x, w0, out0], grid=(2, 2, 1))
    sb.bind_consts("matvec", (32, 8))
    sb.kernel_call("matvec", [out0, w1, out1], grid=(2, 1, 1))
    sb.kernel_call("relu", [out1])
    want = np.maximum((x.astype(np.float64) @ w0) @ w1, 0)
    assert np.abs(out1 - want).max() < 1e-3 * np.abs(want).max()


@pytest.mark.parametrize("m,k", [(64, 8), (33, 36), (257, 200), (1001, 1024), (64, 1032), (50, 77)])
def test_matvec_matches_oracle(sb, oracle, m, k):
    """Register-cached vector path (k % 4 == 0, k <= 1024; odd and even row counts), the long-row
    vector path and the scalar path."""
    x, y = uniform((m, k), 11), uniform(k, 12)
    z = np.zeros(m, np.float32)
    want = np.zeros(m, np.float32)
    sb.bind_consts("matvec", (1, 1))
    sb.kernel_call("matvec", [x, y, z], grid=(m, 1, 1))
    oracle.lib.sile_oracle_bind_matvec(1, 1)
    oracle.launch("matvec", [x, y, want], grid=(m, 1, 1))
    assert np.abs(z - want).max() < 1e-3 * max(np.abs(want).max(), 1e-6)
