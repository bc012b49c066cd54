"""The C-ABI library loads and exports every symbol include/sile_cuda.h declares
(no compute: runs without a GPU)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import sile_b200
    sile_b200.build()
    return sile_b200._lib.lib()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sile_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sile_(?:kernel|cuda)_\w+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    import sile_b200
    declared = _declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in sile_cuda.h but not exported"
    assert set(declared) == set(sile_b200._lib.EXPORTED_SYMBOLS)


def test_version_and_error_string(lib):
    assert lib.sile_cuda_version() >= 100
    assert isinstance(lib.sile_cuda_last_error(), bytes)


def test_status_word_maps_to_timeout_error(lib):
    """The word a kernel leaves after a bounded wait ran out -> code and message, as the blocking
    entry points report it after reading the word back (host-side mapping only: no GPU wait is
    made to run out here)."""
    import sile_b200
    assert lib.sile_cuda_decode_status(0) == sile_b200._lib.OK
    word = sile_b200._lib.ERR_TIMEOUT | (1 << (8 + 3)) | (1 << (8 + 8))
    assert lib.sile_cuda_decode_status(word) == sile_b200._lib.ERR_TIMEOUT
    msg = lib.sile_cuda_last_error()
    assert b"wait ran out" in msg and b"0x108" in msg
    assert lib.sile_cuda_last_status() == sile_b200._lib.ERR_TIMEOUT


def test_slice_plans_of_the_sharded_headline_gemm(lib):
    """Host arithmetic of the sliced GEMM kernel's work plan, for one rank's block of the 8192^3
    GEMM on 74 CTA pairs: 2 GPUs -- whole tiles (a staggered head would add a round); 4 GPUs -- a
    quarter wave cut in two at the head, the last wave cut in two; 8 GPUs (exchange-bound) -- a
    three-phase head (half tiles for two thirds of the pairs, a second half tile for half of
    those), whole tiles after it; one destination -- only the last wave."""
    import ctypes as C

    def plan(tiles, dest, exchange_bound):
        buf = C.create_string_buffer(128)
        assert lib.sile_cuda_gemm_slice_plan(tiles, 74, dest, int(exchange_bound), buf, len(buf)) == 0
        return buf.value.decode()

    assert plan(512, 2, False) == "444x1+68x1"
    assert plan(256, 4, False) == "18x2+222x1+16x2"
    assert plan(128, 8, True) == "24x2+26x1+12x2+66x1"
    assert plan(256, 1, False) == "222x1+34x2"
    assert plan(128, 1, False) == "74x1+54x1"
    for text, tiles in ((plan(t, d, e), t) for t in (1, 73, 74, 75, 300, 1024) for d in (1, 4) for e in (False, True)):
        groups = [tuple(map(int, g.split("x"))) for g in text.split("+")]
        assert sum(n for n, _ in groups) == tiles and all(s in (1, 2, 4) for _, s in groups), text
    assert lib.sile_cuda_gemm_slice_plan(0, 74, 1, 0, C.create_string_buffer(64), 64) != 0


def test_bind_consts_validation(lib):
    import ctypes as C
    import sile_b200
    arr = (C.c_int64 * 3)(2, 2, 2)
    assert lib.sile_cuda_bind_consts(b"matmul", arr, 3) == 0
    assert lib.sile_cuda_bind_consts(b"matmul", arr, 2) == sile_b200._lib.ERR_INVALID
    assert lib.sile_cuda_bind_consts(b"nonesuch", arr, 3) == sile_b200._lib.ERR_UNSUPPORTED
    bad = (C.c_int64 * 3)(2, 0, 2)
    assert lib.sile_cuda_bind_consts(b"matmul", bad, 3) == sile_b200._lib.ERR_INVALID
    assert b"positive" in lib.sile_cuda_last_error()


def test_desc_and_shape_validation_precede_device_use(lib):
    import ctypes as C
    import sile_b200
    d = sile_b200.make_desc(sile_b200._lib.OP_MATMUL)
    d.struct_size = 4
    grid = (C.c_uint32 * 3)(1, 1, 1)
    rc = lib.sile_cuda_launch_host(C.byref(d), None, None, 0, grid)
    assert rc == sile_b200._lib.ERR_INVALID


def test_no_cpu_fallback_without_device(lib):
    """Without a GPU the compute entry points fail loudly instead of computing on the host."""
    import numpy as np
    import torch
    import sile_b200
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    a = np.ones((4, 4), np.float32)
    c = np.zeros((4, 4), np.float32)
    with pytest.raises(sile_b200.SileError) as e:
        sile_b200.kernel_call("matmul", [a, a, c], grid=(4, 1, 1))
    assert e.value.code in (sile_b200._lib.ERR_NO_DEVICE, sile_b200._lib.ERR_CUDA)
    assert (c == 0).all()


def test_product_never_imports_oracle():
    pkg = os.path.join(ROOT, "sile_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"
