"""ctypes loader for the plain-C oracle (test infrastructure only).

The C file restates the reference's generated CPU code; see ``sile_oracle.h``
for which functions are pinned by the reference's golden vectors.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libsile_oracle.so")
_SRC = [os.path.join(_HERE, "sile_oracle.c"), os.path.join(_HERE, "sile_oracle.h")]


def build(force: bool = False) -> str:
    """Compile the oracle with the reference's CPU flags if it is stale."""
    stale = force or not os.path.exists(_SO) or any(
        os.path.getmtime(s) > os.path.getmtime(_SO) for s in _SRC)
    if stale:
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        subprocess.run(
            ["gcc", "-shared", "-fPIC", "-O2", "-fopenmp", _SRC[0], "-o", _SO, "-lm"],
            check=True)
    return _SO


_i64 = C.c_int64
_KERNEL_SIG = [C.POINTER(C.c_void_p), _i64, _i64, C.POINTER(_i64), _i64]


def _fptr(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.POINTER(C.c_float))


class Oracle:
    """Thin numpy front end over the C oracle."""

    def __init__(self, so_path: str | None = None):
        self.lib = C.CDLL(so_path or build())
        L = self.lib
        for name in ("matmul", "vec_add", "relu", "softmax", "parallel_reduce", "matvec"):
            fn = getattr(L, f"sile_kernel_{name}")
            fn.argtypes = _KERNEL_SIG
            fn.restype = None
        L.sile_oracle_bind_matmul.argtypes = [_i64] * 3
        L.sile_oracle_bind_vec_add.argtypes = [_i64]
        L.sile_oracle_bind_softmax.argtypes = [_i64] * 2
        L.sile_oracle_bind_parallel_reduce.argtypes = [_i64]
        L.sile_oracle_bind_matvec.argtypes = [_i64] * 2
        fp = C.POINTER(C.c_float)
        L.sile_oracle_matmul.argtypes = [fp, fp, fp] + [_i64] * 7
        L.sile_oracle_matmul_acc.argtypes = [fp, fp, fp] + [_i64] * 7
        L.sile_oracle_matmul_tiles.argtypes = [fp, fp, fp] + [_i64] * 6 + [C.POINTER(_i64), _i64]
        L.sile_oracle_attention.argtypes = [fp, fp, fp, fp] + [_i64] * 5 + [
            C.c_float, C.c_int, C.POINTER(_i64), _i64]
        L.sile_oracle_num_threads.restype = C.c_int
        L.sile_oracle_set_num_threads.argtypes = [C.c_int]

    # -- exact-ABI launch, as the reference's CPU runtime performs it
    #    (crates/sile-backend/src/cpu/mod.rs:104-128)
    def launch(self, name: str, arrays, grid=(1, 1, 1)) -> None:
        bufs = (C.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
        shapes = [d for a in arrays for d in a.shape]
        sh = (_i64 * len(shapes))(*shapes)
        ntg = int(grid[0]) * int(grid[1]) * int(grid[2])
        getattr(self.lib, f"sile_kernel_{name}")(bufs, ntg, 1, sh, len(shapes))

    def num_threads(self) -> int:
        return int(self.lib.sile_oracle_num_threads())

    def use_all_cores(self) -> int:
        """OpenMP threads = the cores this process may run on, whatever OMP_NUM_THREADS says
        (process launchers such as torch.distributed.run export OMP_NUM_THREADS=1)."""
        try:
            n = len(os.sched_getaffinity(0))
        except AttributeError:
            n = os.cpu_count() or 1
        self.lib.sile_oracle_set_num_threads(n)
        return self.num_threads()

    def matmul(self, a, b, bm, bn, bk, grid=None):
        m, k = a.shape
        n = b.shape[1]
        c = np.zeros((m, n), np.float32)
        ntg = (m // bm) * (n // bn) if grid is None else int(np.prod(grid))
        self.lib.sile_oracle_matmul(_fptr(a), _fptr(b), _fptr(c), m, n, k, bm, bn, bk, ntg)
        return c

    def matmul_acc(self, a, b, c, bm, bn, bk, grid=None):
        """c + a @ b over whole logical tiles (accumulator seeded from c); returns a new array."""
        m, k = a.shape
        n = b.shape[1]
        out = np.ascontiguousarray(c, dtype=np.float32).copy()
        ntg = (m // bm) * (n // bn) if grid is None else int(np.prod(grid))
        self.lib.sile_oracle_matmul_acc(_fptr(a), _fptr(b), _fptr(out), m, n, k, bm, bn, bk, ntg)
        return out

    def matmul_tiles(self, a, b, bm, bn, bk, tile_ids):
        """Compute only the listed logical tiles; the rest of C stays zero."""
        m, k = a.shape
        n = b.shape[1]
        c = np.zeros((m, n), np.float32)
        ids = np.ascontiguousarray(tile_ids, dtype=np.int64)
        self.lib.sile_oracle_matmul_tiles(
            _fptr(a), _fptr(b), _fptr(c), m, n, k, bm, bn, bk,
            ids.ctypes.data_as(C.POINTER(_i64)), ids.size)
        return c

    def attention(self, q, kt, v, bh, s, d, bm, bn, scale, causal, units=None):
        """q,v: [bh*s,d]; kt: [bh*d,s]; returns o [bh*s,d] (only ``units`` filled)."""
        o = np.zeros((bh * s, d), np.float32)
        if units is None:
            up, un = None, 0
        else:
            units = np.ascontiguousarray(units, dtype=np.int64)
            up, un = units.ctypes.data_as(C.POINTER(_i64)), units.size
        self.lib.sile_oracle_attention(_fptr(q), _fptr(kt), _fptr(v), _fptr(o), bh, s, d,
                                       bm, bn, float(scale), int(bool(causal)), up, un)
        return o


_cached = None


def load() -> Oracle:
    global _cached
    if _cached is None:
        _cached = Oracle()
    return _cached
