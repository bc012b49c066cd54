/*
 * libsile_cuda -- B200 (sm_100a) backend for sile's kernel-launch boundary.
 *
 * Plain C ABI: pointers and sizes only.  Two families of entry points:
 *
 *  1. sile_kernel_<name>: the exact signature sile's CPU backend generates and
 *     its runtime dlopen()s and calls (host pointers in, results in place,
 *     complete on return).  A maintainer can point the existing runtime at this
 *     library unchanged.
 *  2. sile_cuda_launch / sile_cuda_launch_host: what a `Device::Cuda` arm of
 *     sile's KernelLauncher::apply would bind -- a kernel description plus
 *     buffers, with dtype/layout extensions the f32-only reference lacks.
 *
 * No entry point falls back to a CPU implementation: without a usable sm_100
 * device every call fails with SILE_ERR_NO_DEVICE / SILE_ERR_CUDA.
 */
#ifndef SILE_CUDA_H
#define SILE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  They mirror sile_core::Error (crates/sile-core/src/error.rs:2-13):
 * INVALID ~ Error::Shape, UNSUPPORTED ~ Error::UnsupportedBackend,
 * NO_DEVICE ~ Error::InvalidDevice, CUDA ~ Error::Io-like runtime failure. */
#define SILE_OK 0
#define SILE_ERR_INVALID 1
#define SILE_ERR_UNSUPPORTED 2
#define SILE_ERR_CUDA 3
#define SILE_ERR_TIMEOUT 4 /* a bounded device-side wait ran out; the context stays usable */
#define SILE_ERR_NO_DEVICE 5

/* Element types.  The reference has F32 only (crates/sile-hir/src/types.rs:11-14);
 * BF16/F16 are surface extensions. */
#define SILE_DTYPE_F32 0
#define SILE_DTYPE_BF16 1
#define SILE_DTYPE_F16 2

/* Layout of the B operand of a matmul.  The reference is row-major only
 * (crates/sile-tile-ir/src/lower.rs:991-1002); COL_MAJOR means B[K,N] stored
 * as [N,K] row-major. */
#define SILE_LAYOUT_ROW_MAJOR 0
#define SILE_LAYOUT_COL_MAJOR 1

/* Kernel patterns the backend recognises.  Each is the hand-written equivalent of
 * one generated unit of the reference (canonical_matmul.rs:24-444 and the per-op
 * loop nests of crates/sile-tile-ir/src/passes/lowering/). */
#define SILE_OP_MATMUL 1          /* examples/matmul.rs:3-18 */
#define SILE_OP_ATTENTION 2       /* composed from mma/reduce_max/exp/reduce_sum tile ops.  Two forms:
                                     16-bit q, k, v, o of one shape [.., S, 128] (rank 2..4); or, with
                                     in/out dtype F32, the reference's rank-2 tensors with K transposed
                                     (see sile_kernel_attention) */
#define SILE_OP_VEC_ADD 3         /* examples/vec_add.rs:3-10 */
#define SILE_OP_RELU 4            /* examples/mlp.rs:51-55 */
#define SILE_OP_SOFTMAX 5         /* examples/softmax.rs:3-16 */
#define SILE_OP_PARALLEL_REDUCE 6 /* examples/parallel_reduce.rs:3-9 */
#define SILE_OP_MATVEC 7          /* examples/mlp.rs:28-46 */

/* SileKernelDesc.flags.
 * SILE_FLAG_ACCUMULATE (matmul): the accumulator is seeded with the output tile instead of
 * `constant(0.0, [BM, BN])`, i.e. C = C + A * B -- the reference's general mma `D = acc + A * B`
 * with `sum0 = acc[r][c]` (crates/sile-tile-ir/src/passes/lowering/tile_compute/mma.rs:25-260),
 * the path a kernel takes there when CanonicalMatmulPlan::detect refuses its non-zero seed
 * (canonical_matmul.rs:446-666).  C is then an input as well as the output. */
#define SILE_FLAG_ACCUMULATE 1

/* C mirror of what sile_hir::Kernel (crates/sile-hir/src/kernel.rs:9-83) tells a
 * backend once its body has been recognised: which pattern, the const-generic
 * values the reference bakes into generated code, and the dtype/layout extensions. */
typedef struct SileKernelDesc {
  uint32_t struct_size; /* sizeof(SileKernelDesc), for forward compatibility */
  int32_t op;           /* SILE_OP_* */
  int32_t in_dtype;     /* SILE_DTYPE_* of the inputs */
  int32_t out_dtype;    /* SILE_DTYPE_* of the output */
  int32_t b_layout;     /* matmul: SILE_LAYOUT_* of B */
  int32_t causal;       /* attention: 1 = key index <= query index */
  float scale;          /* attention: softmax scale applied to Q*K^T */
  int32_t flags;        /* SILE_FLAG_* bits; 0 for the kernels of the reference's examples */
  int64_t consts[4];    /* matmul: BM,BN,BK; vec_add/parallel_reduce: TILE;
                           softmax: BM,BN; matvec: BM,BK; attention over f32 tensors: BM,BN;
                           0 = unspecified (treated as 1) */
} SileKernelDesc;

/* ---- 1. exact reference ABI -------------------------------------------------
 * Replaces the generated `void sile_kernel_<name>(void** buffers,
 * int64_t num_threadgroups, int64_t threads_per_group, const int64_t* shapes,
 * int64_t num_shapes)` (crates/sile-backend/src/cpu/codegen.rs:448-454; caller
 * crates/sile-backend/src/cpu/mod.rs:12,97-128).  Buffers are HOST float
 * pointers in kernel-parameter order; shapes is the concatenation of every
 * argument's shape; the call stages host<->device and is complete on return.
 * The ABI returns void, as the reference's does: failures are reported through
 * sile_cuda_last_status() / sile_cuda_last_error() and leave outputs untouched. */
void sile_kernel_matmul(void** buffers, int64_t num_threadgroups, int64_t threads_per_group,
                        const int64_t* shapes, int64_t num_shapes);
/* matmul whose accumulator starts from the output tile (SILE_FLAG_ACCUMULATE): buffers a, b, c
 * with c read and written; const generics bound under the name "matmul_acc". */
void sile_kernel_matmul_acc(void** buffers, int64_t num_threadgroups, int64_t threads_per_group,
                            const int64_t* shapes, int64_t num_shapes);
void sile_kernel_vec_add(void** buffers, int64_t num_threadgroups, int64_t threads_per_group,
                         const int64_t* shapes, int64_t num_shapes);
void sile_kernel_relu(void** buffers, int64_t num_threadgroups, int64_t threads_per_group,
                      const int64_t* shapes, int64_t num_shapes);
void sile_kernel_softmax(void** buffers, int64_t num_threadgroups, int64_t threads_per_group,
                         const int64_t* shapes, int64_t num_shapes);
void sile_kernel_parallel_reduce(void** buffers, int64_t num_threadgroups, int64_t threads_per_group,
                                 const int64_t* shapes, int64_t num_shapes);
void sile_kernel_matvec(void** buffers, int64_t num_threadgroups, int64_t threads_per_group,
                        const int64_t* shapes, int64_t num_shapes);
/* Attention forward as the reference's tile ops compose it (load_tile, mma, reduce_max, max_tile,
 * exp, reduce_sum, broadcast, div: crates/sile-tile-ir/src/lower.rs:509-748; general mma
 * crates/sile-tile-ir/src/passes/lowering/tile_compute/mma.rs:25-260), over the reference's tensor
 * model -- f32, rank 2, row-major (crates/sile-hir/src/types.rs:11-14) -- with K given TRANSPOSED
 * because `mma` takes [BM,K] x [K,BN] tiles and the DSL has no transpose op:
 *   buffers = q [BH*S, D], kt [BH*D, S], v [BH*S, D], o [BH*S, D];  shapes = those eight extents.
 * One logical tile = BM query rows of one head; tiles [0, grid product) run
 * (crates/sile-backend/src/cpu/codegen.rs:517-533), the rest of o is left untouched.  Const
 * generics bound under the name "attention": BM, BN, causal (0/1; a surface extension, the DSL
 * has no index tile to build a mask from); the softmax scale, a literal in the kernel body, is
 * bound with sile_cuda_bind_scale.  D must be 128; S must be a multiple of BM and of BN (a query
 * tile may not straddle heads, and the composed kernel's key loop would drop a BN remainder).
 * The tensor cores run in bf16 with f32 accumulation: q, kt, v are rounded to bf16 on the
 * device, so results carry the 2e-2 tolerance of the 16-bit configurations, not 1e-3. */
void sile_kernel_attention(void** buffers, int64_t num_threadgroups, int64_t threads_per_group,
                           const int64_t* shapes, int64_t num_shapes);

/* The reference bakes const generics (tile sizes) into each generated kernel
 * (crates/sile-tile-ir/src/lower.rs:9-34); the exact ABI has no slot for them.
 * This binds them for subsequent sile_kernel_<name> calls from the calling
 * thread.  `name` is the kernel name without the "sile_kernel_" prefix. */
int sile_cuda_bind_consts(const char* name, const int64_t* consts, int64_t num_consts);

/* A float literal of a kernel body that the exact ABI has no slot for either: the softmax scale
 * of "attention" (a constant tile in the reference's DSL, crates/sile-tile-ir/src/lower.rs:509-524).
 * Bound per calling thread like the const generics. */
int sile_cuda_bind_scale(const char* name, float scale);

/* ---- 2. Device::Cuda launch ---------------------------------------------------
 * The arm crates/sile/src/kernel_launcher.rs:69-71 leaves unimplemented, shaped
 * after the one GPU precedent, MetalBackend::execute_llir(func, param_kinds,
 * args, launch, stream) (crates/sile-backend/src/metal/mod.rs:65-76).
 * dev_buffers are DEVICE pointers in kernel-parameter order; shapes as above;
 * grid is LaunchConfig::grid (crates/sile-core/src/kernel.rs:4-6) -- only its
 * product matters, as in cpu/mod.rs:109-120; stream is a cudaStream_t (NULL =
 * default stream).  Asynchronous: returns after enqueueing. */
int sile_cuda_launch(const SileKernelDesc* desc, void* const* dev_buffers, const int64_t* shapes,
                     int64_t num_shapes, const uint32_t grid[3], void* stream);

/* Same launch with HOST buffers: stages inputs to the device, runs, copies
 * outputs (the last buffer; for relu the only buffer) back, and returns when
 * complete -- what MetalBackend::execute_llir does around its dispatch
 * (crates/sile-backend/src/metal/mod.rs:117-125,160-169).  Large 16-bit
 * matmuls with a column-major B are streamed: B first, then A in row chunks
 * (1024 rows; SILE_CUDA_HOST_CHUNK_ROWS overrides) whose GEMMs and copies back
 * overlap the copies in; the streams used are kept per host thread. */
int sile_cuda_launch_host(const SileKernelDesc* desc, void* const* host_buffers, const int64_t* shapes,
                          int64_t num_shapes, const uint32_t grid[3]);

/* ---- multi-GPU sharding ---------------------------------------------------------
 * No counterpart in the reference (single process, single device,
 * crates/sile-core/src/stream.rs:4-19).  A matmul splits by output-column block:
 * the rank owning columns [n_begin, n_begin + n_count) computes
 * C[:, n_begin : n_begin+n_count] = A * B[:, n_begin : n_begin+n_count].
 * `b_shard` is that block of a column-major B ([n_count, K] contiguous); `c` is
 * the base of a row-major buffer with `n_total` columns (pass n_total = n_count
 * and n_begin = 0 for a packed shard buffer).  Asynchronous on `stream`.
 * SILE_FLAG_ACCUMULATE is refused (SILE_ERR_UNSUPPORTED). */
int sile_cuda_matmul_shard(const SileKernelDesc* desc, const void* a, const void* b_shard, void* c,
                           int64_t m, int64_t n_total, int64_t k, int64_t n_begin, int64_t n_count,
                           void* stream);

/* Diagnostic, host arithmetic only (no device needed): how the sliced 256 x 256 GEMM kernel
 * would cut `tiles` tiles over `cta_pairs` resident CTA pairs when storing to `destinations`
 * buffers, as text -- groups of "tiles x slices per tile", e.g. "18x2+222x1+16x2".
 * `exchange_bound` != 0: the peers' share of the output takes longer to cross NVLink than the
 * tiles take to compute.  No counterpart in the reference. */
int sile_cuda_gemm_slice_plan(int32_t tiles, int32_t cta_pairs, int32_t destinations,
                              int32_t exchange_bound, char* out, int64_t capacity);

/* The same column-block matmul with the all-gather folded into its epilogue: rank
 * `rank` of `world` (<= 8) computes its block and stores every element into the
 * full [M, n_total] row-major buffer of EVERY rank.  c_peers[i] is the base of
 * rank i's buffer as mapped into this process (for instance the buffer_ptrs of
 * a torch symmetric-memory allocation; c_peers[rank] is the local one).  Whole tiles leave the
 * epilogue as TMA stores, one per 32-row x 128-byte box and destination (the peers' over NVLink),
 * ragged or launch-masked tiles as st.global from the epilogue warps; the kernel waits on no
 * other GPU.  When the call has completed on every rank and the ranks have synchronised (the
 * caller's barrier), each holds the whole C.  16-bit operands, column-major B, N divisible by
 * world, M > 128.  The 256 x 256 CTA-pair kernel with sliced tiles built for this epilogue
 * runs (stores drain under the next tile; 16-bit and f32 outputs).  SILE_FLAG_ACCUMULATE is
 * refused here. */
int sile_cuda_matmul_allgather(const SileKernelDesc* desc, const void* a, const void* b_shard,
                               void* const* c_peers, int32_t world, int32_t rank, int64_t m,
                               int64_t n_total, int64_t k, void* stream);

/* Attention forward over this rank's slab of heads with the all-gather of O folded into the
 * kernel's epilogue: rank `rank` of `world` (<= 8) holds q, k, v for heads
 * [rank * bh_local, (rank + 1) * bh_local) as [bh_local, S, 128] bf16 and every CTA stores its
 * rows of O (TMA stores, full 128-byte lines) into the [world * bh_local, S, 128] buffer of
 * EVERY rank.  o_peers[i] is the base of rank i's buffer as mapped into this process
 * (o_peers[rank] is the local one).  The kernel waits on no other GPU; when the call has
 * completed on every rank and the ranks have synchronised, each holds the whole O in its final
 * layout.  desc: op SILE_OP_ATTENTION, bf16 in and out, `scale`, `causal`.  The reference shards
 * nothing; this follows the batch x head split with one all-gather of the outputs. */
int sile_cuda_attention_allgather(const SileKernelDesc* desc, const void* q, const void* k,
                                  const void* v, void* const* o_peers, int32_t world, int32_t rank,
                                  int64_t bh_local, int64_t s, void* stream);

/* Lays the rank-major result of an all-gather of packed column blocks,
 * src[parts][rows][cols], out as one row-major matrix dst[rows][parts*cols].
 * `dtype` is a SILE_DTYPE_* giving the element size. */
int sile_cuda_unshard_columns(void* dst, const void* src, int64_t parts, int64_t rows, int64_t cols,
                              int32_t dtype, void* stream);

/* ---- f32 matmul that allocates nothing -------------------------------------------
 * Has no counterpart in the reference.  For callers that cannot let a library
 * allocate device memory -- a process whose own arena already owns all of HBM, a
 * latency-critical loop that must stay clear of the driver's allocation lock and
 * the device-wide synchronisation an allocation can imply, or a deployment that
 * forbids allocation after start-up.  Same result as an f32 SILE_OP_MATMUL through
 * sile_cuda_launch with the full logical grid: C[M,N] = A[M,K] * B[K,N], all
 * row-major f32 DEVICE buffers, logical tile (bm, bn, bk) deciding which part of C
 * is written (0 = 1).
 *
 * The bf16 split planes the kernel needs live in a 32 MiB array that is part of
 * the library image (every GPU that loads the library holds those 32 MiB until
 * the process exits), so the problem must satisfy
 *     4 * (M + N) * roundup(K, 64) bytes <= 32 MiB
 * (e.g. M = N = 1024 with K = 4096, or M = N = 2048 with K = 2048); anything larger
 * is rejected with SILE_ERR_UNSUPPORTED and a message naming the size.  The call
 * makes no cudaMalloc / cudaFree / stream-ordered allocation, here or in anything
 * it calls.
 *
 * The first call on each device resolves the array's device address and sets a
 * kernel attribute; make that first call before any stream capture begins.
 * All calls on a device share the one array: it still holds the previous call's
 * planes when the next call starts (every plane element is rewritten before it is
 * read), and two calls whose kernels can overlap on the GPU -- different streams,
 * or different host threads -- race on it.  Serialise them on one stream.
 *
 * Asynchronous on `stream` when `wait` is 0.  With `wait` != 0 the call returns
 * after the stream has drained and reports SILE_ERR_TIMEOUT if a bounded
 * device-side wait ran out during this (or an earlier non-waiting) call.  After
 * non-waiting calls, sile_cuda_synchronize / sile_cuda_memcpy_d2h report and
 * clear such a time-out too; until one of them (or a waiting call) has read it,
 * every further launch on the device gives up at its first wait, so synchronise
 * through this library before trusting results of a run of non-waiting calls. */
int sile_cuda_matmul_f32_noalloc(const float* a, const float* b, float* c, int64_t m, int64_t n,
                                 int64_t k, int64_t bm, int64_t bn, int64_t bk, void* stream,
                                 int32_t wait);

/* Device selection, after Device::cuda(index) (crates/sile-core/src/device.rs:23-35).
 * Fails with SILE_ERR_NO_DEVICE when the index does not name an sm_100 GPU. */
int sile_cuda_set_device(int index);
int sile_cuda_device_count(void);

/* Stream::synchronize (crates/sile-core/src/stream.rs:17-19), a no-op in the
 * reference, is real here.  Also reports a device-side time-out recorded since
 * the last call (SILE_ERR_TIMEOUT) by any launch of this library on the current
 * device, sile_cuda_matmul_f32_noalloc included, and clears it. */
int sile_cuda_synchronize(void* stream);

/* The error a kernel's status word stands for: low byte = SILE_ERR_* code, bit 8 + n set = wait
 * site n was stuck when the kernel gave up.  Records the message for sile_cuda_last_error() and
 * returns the code; 0 maps to SILE_OK and leaves the last error alone.  Needs no device (the
 * mapping the blocking entry points apply after reading the word back). */
int sile_cuda_decode_status(int status_word);

/* Device-resident tensors and real streams.  The reference's Tensor is a host Vec<f32> and every
 * GPU backend re-uploads it per launch (crates/sile/src/tensor.rs:5-9;
 * crates/sile-backend/src/metal/mod.rs:117-125); with these a binding keeps tensors on the device,
 * launches through sile_cuda_launch on a stream and copies only at Tensor::from_vec / to_vec.
 * No counterpart in the reference.  Buffers are cudaMalloc allocations (256-byte aligned) of the
 * current device; copies are ordered on `stream` and complete on return (the host side is pageable
 * memory); sile_cuda_memcpy_d2h also reports a device-side time-out like sile_cuda_synchronize. */
int sile_cuda_malloc(void** dev_ptr, size_t bytes);
int sile_cuda_free(void* dev_ptr);
int sile_cuda_memcpy_h2d(void* dev_dst, const void* host_src, size_t bytes, void* stream);
int sile_cuda_memcpy_d2h(void* host_dst, const void* dev_src, size_t bytes, void* stream);
int sile_cuda_memset(void* dev_dst, int byte_value, size_t bytes, void* stream);
int sile_cuda_stream_create(void** stream);
int sile_cuda_stream_destroy(void* stream);

/* Scratch the f32 matmul needs on the device for a given problem, in bytes
 * (0 for 16-bit inputs).  sile_cuda_launch obtains it from the stream-ordered
 * allocator itself; the figure is exposed for capacity planning. */
size_t sile_cuda_matmul_workspace_bytes(int64_t m, int64_t n, int64_t k, int32_t in_dtype);

/* Message / code of the calling thread's most recent failure ("" / SILE_OK if none). */
const char* sile_cuda_last_error(void);
int sile_cuda_last_status(void);

/* The kernel the calling thread's most recent launch chose, with its geometry:
 * "<kernel name> grid=<CTAs> block=<threads> smem=<bytes>" ("" before any launch).  The
 * reference prints the generated source / IR of every launch to stderr under SILE_PRINT_SOURCE,
 * SILE_PRINT_LLVMIR, SILE_PRINT_TILEIR (crates/sile/src/kernel_launcher.rs:11-13,48-53); with
 * any of the three set this library prints the same line per launch instead -- its kernels are
 * hand-written, so the choice and geometry are what there is to dump. */
const char* sile_cuda_last_kernel(void);

/* Library version: major*10000 + minor*100 + patch. */
int sile_cuda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SILE_CUDA_H */
