"""sile_b200: sm_100a kernels behind sile's kernel-launch boundary.

The product is ``lib/libsile_cuda.so`` (C ABI in ``include/sile_cuda.h``); this package
is the thin Python front end the tests and the bench use to reach it."""
from . import _lib, api  # noqa: F401
from .api import (KernelLauncher, SileError, attention, attention_allgather, attention_f32, bind_consts, bind_scale,  # noqa: F401
                  kernel_call, make_desc, matmul, matmul_allgather, matmul_shard, matvec, parallel_reduce, relu, softmax,
                  synchronize, unshard_columns, vec_add)
from .build import build  # noqa: F401

__all__ = ["KernelLauncher", "SileError", "attention", "attention_allgather", "attention_f32", "bind_consts", "bind_scale",
           "kernel_call", "make_desc",
           "matmul", "matvec", "parallel_reduce", "relu", "softmax", "synchronize", "vec_add", "build"]
