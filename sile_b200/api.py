"""Python front end over the C ABI, used by the tests and the bench.

It mirrors the reference's launch surface -- ``kernel(args...).grid((x, y, z)).apply(stream)``
(crates/sile/src/kernel_launcher.rs:15-74) -- with torch tensors standing in for the
reference's host ``Tensor`` (crates/sile/src/tensor.rs:27-88).  torch is used for device
memory and streams only; all compute goes through libsile_cuda.so.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

from . import _lib
from ._lib import (DTYPE_BF16, DTYPE_F16, DTYPE_F32, LAYOUT_COL_MAJOR, LAYOUT_ROW_MAJOR,
                   OP_ATTENTION, OP_MATMUL, OP_MATVEC, OP_PARALLEL_REDUCE, OP_RELU, OP_SOFTMAX,
                   OP_VEC_ADD, KernelDesc)


class SileError(RuntimeError):
    """Counterpart of sile_core::Error (crates/sile-core/src/error.rs:2-13)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[sile_cuda status {code}] {message}")
        self.code = code


def _check(rc: int) -> None:
    if rc != _lib.OK:
        raise SileError(rc, _lib.lib().sile_cuda_last_error().decode())


def _dtype_code(t) -> int:
    import torch
    return {torch.float32: DTYPE_F32, torch.bfloat16: DTYPE_BF16, torch.float16: DTYPE_F16}[t.dtype]


def make_desc(op: int, in_dtype=DTYPE_F32, out_dtype=DTYPE_F32, b_layout=LAYOUT_ROW_MAJOR,
              causal=False, scale=1.0, consts: Sequence[int] = (), flags: int = 0) -> KernelDesc:
    d = KernelDesc()
    d.struct_size = C.sizeof(KernelDesc)
    d.op, d.in_dtype, d.out_dtype, d.b_layout = op, in_dtype, out_dtype, b_layout
    d.causal, d.scale, d.flags = int(bool(causal)), float(scale), int(flags)
    for i, v in enumerate(consts):
        d.consts[i] = int(v)
    return d


class KernelLauncher:
    """``kernel(args...).grid(g).apply(stream)`` over device tensors (async on the stream)."""

    def __init__(self, desc: KernelDesc, args):
        self.desc, self.args, self._grid = desc, list(args), (1, 1, 1)

    def grid(self, g):
        g = tuple(int(x) for x in g) + (1, 1, 1)
        self._grid = g[:3]
        return self

    def apply(self, stream=None):
        import torch
        bufs = (C.c_void_p * len(self.args))(*[t.data_ptr() for t in self.args])
        shapes = [int(d) for t in self.args for d in t.shape]
        sh = (C.c_int64 * len(shapes))(*shapes)
        grid = (C.c_uint32 * 3)(*self._grid)
        if stream is None:
            stream = torch.cuda.current_stream()
        handle = stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)
        _check(_lib.lib().sile_cuda_launch(C.byref(self.desc), bufs, sh, len(shapes), grid, C.c_void_p(handle)))
        return self

    def apply_host(self):
        """Blocking launch over HOST buffers (numpy arrays or CPU torch tensors)."""
        ptrs, shapes = [], []
        for t in self.args:
            ptrs.append(t.data_ptr() if hasattr(t, "data_ptr") else t.ctypes.data)
            shapes += [int(d) for d in t.shape]
        bufs = (C.c_void_p * len(ptrs))(*ptrs)
        sh = (C.c_int64 * len(shapes))(*shapes)
        grid = (C.c_uint32 * 3)(*self._grid)
        _check(_lib.lib().sile_cuda_launch_host(C.byref(self.desc), bufs, sh, len(shapes), grid))
        return self


def _full_grid(m, n, bm, bn):
    return (max(m // bm, 1), max(n // bn, 1), 1)


def matmul(a, b, c, bm=1, bn=1, bk=1, b_layout=LAYOUT_ROW_MAJOR, accumulate=False) -> KernelLauncher:
    """``matmul::<BM,BN,BK>(&a, &b, &mut c)`` (crates/sile/examples/matmul.rs:3-18).

    With ``b_layout=LAYOUT_COL_MAJOR`` ``b`` is given as an [N, K] row-major tensor.  With
    ``accumulate`` the accumulator is seeded with ``c``'s tile (``c = c + a @ b``), the general
    ``mma(a, b, acc)`` of crates/sile-tile-ir/src/passes/lowering/tile_compute/mma.rs:25-260."""
    import torch
    if b_layout == LAYOUT_COL_MAJOR:
        # the ABI carries logical shapes: b is [K, N]
        class _View:
            def __init__(self, t):
                self._t, self.shape = t, (t.shape[1], t.shape[0])

            def data_ptr(self):
                return self._t.data_ptr()
        b_arg = _View(b)
    else:
        b_arg = b
    in_dt = _dtype_code(a) if isinstance(a, torch.Tensor) else DTYPE_F32
    out_dt = _dtype_code(c) if isinstance(c, torch.Tensor) else DTYPE_F32
    desc = make_desc(OP_MATMUL, in_dt, out_dt, b_layout, consts=(bm, bn, bk),
                     flags=_lib.FLAG_ACCUMULATE if accumulate else 0)
    kl = KernelLauncher(desc, [a, b_arg, c])
    return kl.grid(_full_grid(c.shape[0], c.shape[1], bm, bn))


def attention(q, k, v, o, scale: float, causal: bool = False) -> KernelLauncher:
    """Fused attention forward over [.., S, D] bf16 tensors (batch and head dims leading)."""
    desc = make_desc(OP_ATTENTION, _dtype_code(q), _dtype_code(o), causal=causal, scale=scale)
    return KernelLauncher(desc, [q, k, v, o]).grid((q.numel() // (q.shape[-1] * q.shape[-2]), 1, 1))


def attention_f32(q, kt, v, o, bm: int, bn: int, scale: float, causal: bool = False) -> KernelLauncher:
    """Attention over the reference's own tensor model: f32 rank-2 ``q [BH*S, D]``, ``kt [BH*D, S]``
    (K transposed: the DSL's ``mma`` takes [BM,K] x [K,BN] tiles and has no transpose), ``v``, ``o``
    ``[BH*S, D]``; one logical tile = ``bm`` query rows.  Device or host buffers."""
    desc = make_desc(OP_ATTENTION, DTYPE_F32, DTYPE_F32, causal=causal, scale=scale, consts=(bm, bn))
    return KernelLauncher(desc, [q, kt, v, o]).grid((q.shape[0] // bm, 1, 1))


def bind_scale(name: str, scale: float) -> None:
    _check(_lib.lib().sile_cuda_bind_scale(name.encode(), C.c_float(scale)))


def vec_add(a, b, c, tile=4) -> KernelLauncher:
    return KernelLauncher(make_desc(OP_VEC_ADD, consts=(tile,)), [a, b, c]).grid((a.shape[0] // tile, 1, 1))


def relu(x) -> KernelLauncher:
    return KernelLauncher(make_desc(OP_RELU), [x]).grid((1, 1, 1))


def softmax(x, y, bm=1, bn=None) -> KernelLauncher:
    """``softmax::<BM,BN>(&x, &mut y)`` (crates/sile/examples/softmax.rs:3-16): every [bm, bn] tile is
    normalised on its own; ``bn`` defaults to the whole row."""
    bn = x.shape[1] if bn is None else bn
    return KernelLauncher(make_desc(OP_SOFTMAX, consts=(bm, bn)), [x, y]).grid((x.shape[0] // bm, max(x.shape[1] // bn, 1), 1))


def parallel_reduce(a, out, tile=1) -> KernelLauncher:
    return KernelLauncher(make_desc(OP_PARALLEL_REDUCE, consts=(tile,)), [a, out]).grid((a.shape[0] // tile, 1, 1))


def matvec(x, y, z, bm=1, bk=1) -> KernelLauncher:
    return KernelLauncher(make_desc(OP_MATVEC, consts=(bm, bk)), [x, y, z]).grid((x.shape[0] // bm, 1, 1))


def bind_consts(name: str, consts: Sequence[int]) -> None:
    arr = (C.c_int64 * len(consts))(*[int(c) for c in consts])
    _check(_lib.lib().sile_cuda_bind_consts(name.encode(), arr, len(consts)))


def kernel_call(name: str, arrays, grid=(1, 1, 1)) -> None:
    """The reference runtime's call of ``sile_kernel_<name>`` on HOST float buffers
    (crates/sile-backend/src/cpu/mod.rs:104-128).  Raises if the library recorded a failure."""
    L = _lib.lib()
    bufs = (C.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    shapes = [int(d) for a in arrays for d in a.shape]
    sh = (C.c_int64 * len(shapes))(*shapes)
    ntg = int(grid[0]) * int(grid[1]) * int(grid[2])
    getattr(L, f"sile_kernel_{name}")(bufs, ntg, 1, sh, len(shapes))
    rc = L.sile_cuda_last_status()
    if rc != _lib.OK:
        raise SileError(rc, L.sile_cuda_last_error().decode())


def synchronize(stream=None) -> None:
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    _check(_lib.lib().sile_cuda_synchronize(C.c_void_p(stream.cuda_stream)))


def _stream_handle(stream):
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))


def matmul_shard(a, b_shard, c, n_begin: int, n_total: int, bm=1, bn=1, bk=1, stream=None) -> None:
    """One rank's column block of a sharded matmul: ``c[:, n_begin:n_begin+n_count] = a @ B_block``.

    ``b_shard`` is the [n_count, K] block of a column-major B; ``c`` is the base of a row-major
    buffer with ``n_total`` columns (``n_total == n_count`` for a packed shard buffer)."""
    desc = make_desc(OP_MATMUL, _dtype_code(a), _dtype_code(c), LAYOUT_COL_MAJOR, consts=(bm, bn, bk))
    m, k = a.shape
    _check(_lib.lib().sile_cuda_matmul_shard(C.byref(desc), a.data_ptr(), b_shard.data_ptr(), c.data_ptr(),
                                             m, n_total, k, n_begin, b_shard.shape[0], _stream_handle(stream)))


def unshard_columns(dst, src, stream=None) -> None:
    """``dst[r, j*cols + c] = src[j, r, c]`` for the gathered ``src`` of shape [parts, rows, cols]."""
    parts, rows, cols = src.shape
    _check(_lib.lib().sile_cuda_unshard_columns(dst.data_ptr(), src.data_ptr(), parts, rows, cols,
                                                _dtype_code(src), _stream_handle(stream)))


def attention_allgather(q, k, v, o_ptrs, rank: int, scale: float, causal: bool = False, stream=None) -> None:
    """Attention forward over this rank's heads whose epilogue stores O into every rank's buffer.

    ``q, k, v`` are this rank's [bh_local, S, 128] bf16 slabs; ``o_ptrs`` lists the device address
    of each rank's [world * bh_local, S, 128] bf16 buffer as mapped into this process
    (``o_ptrs[rank]`` is the local one)."""
    desc = make_desc(OP_ATTENTION, _dtype_code(q), DTYPE_BF16, causal=causal, scale=scale)
    bh_local = q.numel() // (q.shape[-1] * q.shape[-2])
    arr = (C.c_void_p * len(o_ptrs))(*[int(p) for p in o_ptrs])
    _check(_lib.lib().sile_cuda_attention_allgather(C.byref(desc), q.data_ptr(), k.data_ptr(), v.data_ptr(), arr, len(o_ptrs), rank,
                                                    bh_local, q.shape[-2], _stream_handle(stream)))


def matmul_allgather(a, b_shard, c_ptrs, rank: int, n_total: int, out_dtype, bm=1, bn=1, bk=1, stream=None) -> None:
    """Column-block matmul whose epilogue stores the block into every rank's full C.

    ``c_ptrs`` lists the device addresses of each rank's [M, n_total] buffer as mapped into
    this process (``c_ptrs[rank]`` is the local one); ``out_dtype`` is a torch dtype."""
    import torch
    code = {torch.float32: DTYPE_F32, torch.bfloat16: DTYPE_BF16, torch.float16: DTYPE_F16}[out_dtype]
    desc = make_desc(OP_MATMUL, _dtype_code(a), code, LAYOUT_COL_MAJOR, consts=(bm, bn, bk))
    m, k = a.shape
    arr = (C.c_void_p * len(c_ptrs))(*[int(p) for p in c_ptrs])
    _check(_lib.lib().sile_cuda_matmul_allgather(C.byref(desc), a.data_ptr(), b_shard.data_ptr(), arr, len(c_ptrs), rank,
                                                 m, n_total, k, _stream_handle(stream)))
