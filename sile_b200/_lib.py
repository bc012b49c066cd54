"""ctypes binding of libsile_cuda.so (the C ABI declared in include/sile_cuda.h).

There is no fallback: if the shared library is missing, loading raises."""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_NO_DEVICE = range(6)
DTYPE_F32, DTYPE_BF16, DTYPE_F16 = 0, 1, 2
LAYOUT_ROW_MAJOR, LAYOUT_COL_MAJOR = 0, 1
FLAG_ACCUMULATE = 1
OP_MATMUL, OP_ATTENTION, OP_VEC_ADD, OP_RELU, OP_SOFTMAX, OP_PARALLEL_REDUCE, OP_MATVEC = range(1, 8)

# Every symbol include/sile_cuda.h declares.
EXPORTED_SYMBOLS = (
    "sile_kernel_matmul", "sile_kernel_matmul_acc", "sile_kernel_vec_add", "sile_kernel_relu", "sile_kernel_softmax",
    "sile_kernel_parallel_reduce", "sile_kernel_matvec", "sile_kernel_attention", "sile_cuda_bind_consts", "sile_cuda_bind_scale",
    "sile_cuda_launch", "sile_cuda_launch_host", "sile_cuda_matmul_shard",
    "sile_cuda_matmul_allgather", "sile_cuda_attention_allgather", "sile_cuda_unshard_columns", "sile_cuda_matmul_f32_noalloc", "sile_cuda_set_device", "sile_cuda_gemm_slice_plan",
    "sile_cuda_device_count", "sile_cuda_synchronize", "sile_cuda_decode_status", "sile_cuda_malloc", "sile_cuda_free",
    "sile_cuda_memcpy_h2d", "sile_cuda_memcpy_d2h", "sile_cuda_memset", "sile_cuda_stream_create",
    "sile_cuda_stream_destroy", "sile_cuda_matmul_workspace_bytes",
    "sile_cuda_last_error", "sile_cuda_last_status", "sile_cuda_last_kernel", "sile_cuda_version",
)


class KernelDesc(C.Structure):
    """Mirror of SileKernelDesc."""
    _fields_ = [
        ("struct_size", C.c_uint32), ("op", C.c_int32), ("in_dtype", C.c_int32),
        ("out_dtype", C.c_int32), ("b_layout", C.c_int32), ("causal", C.c_int32),
        ("scale", C.c_float), ("flags", C.c_int32), ("consts", C.c_int64 * 4),
    ]


_i64 = C.c_int64
_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("SILE_CUDA_LIBRARY", LIB_PATH)  # an alternative build of the same library
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m sile_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    L = C.CDLL(path)
    ksig = [C.POINTER(C.c_void_p), _i64, _i64, C.POINTER(_i64), _i64]
    for name in EXPORTED_SYMBOLS:
        if name.startswith("sile_kernel_"):
            fn = getattr(L, name)
            fn.argtypes, fn.restype = ksig, None
    L.sile_cuda_bind_consts.argtypes = [C.c_char_p, C.POINTER(_i64), _i64]
    L.sile_cuda_bind_scale.argtypes = [C.c_char_p, C.c_float]
    L.sile_cuda_launch.argtypes = [C.POINTER(KernelDesc), C.POINTER(C.c_void_p), C.POINTER(_i64), _i64,
                                   C.POINTER(C.c_uint32), C.c_void_p]
    L.sile_cuda_launch_host.argtypes = [C.POINTER(KernelDesc), C.POINTER(C.c_void_p), C.POINTER(_i64), _i64,
                                        C.POINTER(C.c_uint32)]
    L.sile_cuda_matmul_shard.argtypes = [C.POINTER(KernelDesc), C.c_void_p, C.c_void_p, C.c_void_p,
                                         _i64, _i64, _i64, _i64, _i64, C.c_void_p]
    L.sile_cuda_gemm_slice_plan.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_char_p, C.c_int64]
    L.sile_cuda_gemm_slice_plan.restype = C.c_int
    L.sile_cuda_matmul_allgather.argtypes = [C.POINTER(KernelDesc), C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p),
                                             C.c_int32, C.c_int32, _i64, _i64, _i64, C.c_void_p]
    L.sile_cuda_attention_allgather.argtypes = [C.POINTER(KernelDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p),
                                                C.c_int32, C.c_int32, _i64, _i64, C.c_void_p]
    L.sile_cuda_unshard_columns.argtypes = [C.c_void_p, C.c_void_p, _i64, _i64, _i64, C.c_int32, C.c_void_p]
    L.sile_cuda_matmul_f32_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p] + [_i64] * 6 + [C.c_void_p, C.c_int32]
    L.sile_cuda_set_device.argtypes = [C.c_int]
    L.sile_cuda_synchronize.argtypes = [C.c_void_p]
    L.sile_cuda_decode_status.argtypes = [C.c_int]
    L.sile_cuda_malloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t]
    L.sile_cuda_free.argtypes = [C.c_void_p]
    L.sile_cuda_memcpy_h2d.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    L.sile_cuda_memcpy_d2h.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    L.sile_cuda_memset.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]
    L.sile_cuda_stream_create.argtypes = [C.POINTER(C.c_void_p)]
    L.sile_cuda_stream_destroy.argtypes = [C.c_void_p]
    L.sile_cuda_matmul_workspace_bytes.argtypes = [_i64, _i64, _i64, C.c_int32]
    L.sile_cuda_matmul_workspace_bytes.restype = C.c_size_t
    L.sile_cuda_last_error.restype = C.c_char_p
    L.sile_cuda_last_kernel.restype = C.c_char_p
    _lib = L
    return L
