// extern "C" surface of libsile_cuda.so (declared in include/sile_cuda.h).
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "internal.h"

namespace sile {
namespace {

thread_local std::string t_last_error;
thread_local int t_last_status = SILE_OK;

// Const generics bound for the exact-ABI entry points, per calling thread.
struct BoundConsts {
  int64_t matmul[3] = {1, 1, 1};
  int64_t matmul_acc[3] = {1, 1, 1};
  int64_t vec_add[1] = {4};  // the tile the reference's example hard-codes (examples/vec_add.rs:6)
  int64_t softmax[2] = {1, 0};  // BN = 0: whole row
  int64_t parallel_reduce[1] = {1};
  int64_t matvec[2] = {1, 1};
  int64_t attention[3] = {1, 1, 0};  // BM, BN, causal
  float attention_scale = 1.0f;
};
thread_local BoundConsts t_consts;

std::mutex g_status_mutex;
int* g_status_words[64] = {nullptr};
constexpr int kWorkCounters = 1024;
int* g_work_counters[64] = {nullptr};
unsigned g_work_counter_next[64] = {0};

thread_local char t_last_kernel[160] = "";

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;
std::once_flag g_encode_once;

int check_device() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(SILE_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
  }
  static thread_local int checked_dev = -1;
  if (checked_dev == dev) return SILE_OK;
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(SILE_ERR_NO_DEVICE, "cannot query device %d: %s", dev, cudaGetErrorString(e));
  }
  if (major != 10) return fail(SILE_ERR_NO_DEVICE, "device %d is sm_%d0; this library is built for sm_100a only", dev, major);
  checked_dev = dev;
  return SILE_OK;
}

}  // namespace

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_last_error = buf;
  t_last_status = code;
  return code;
}

int decode_status_word(int word) {
  if (word == 0) return SILE_OK;
  return fail(word & 0xff, "a device-side wait ran out (code %d, stuck wait sites 0x%x); results of the affected launch are invalid",
              word & 0xff, static_cast<unsigned>(word) >> 8);
}

int device_status_word(int** out) {
  int dev = 0;
  SILE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SILE_ERR_INVALID, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status_words[dev]) {
    int* p = nullptr;
    SILE_CUDA_TRY(cudaMalloc(&p, sizeof(int)));
    SILE_CUDA_TRY(cudaMemset(p, 0, sizeof(int)));
    g_status_words[dev] = p;
  }
  *out = g_status_words[dev];
  return SILE_OK;
}

// Staging buffers and workspaces come from a memory pool of the library's own (one per device),
// which keeps what is freed for the next call; the application's default pool is left alone.
cudaMemPool_t g_pools[64] = {nullptr};

int pool_alloc(void** ptr, size_t bytes, cudaStream_t stream) {
  int dev = 0;
  SILE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SILE_ERR_INVALID, "device index %d out of range", dev);
  cudaMemPool_t pool = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_pools[dev]) {
      cudaMemPoolProps props = {};
      props.allocType = cudaMemAllocationTypePinned;
      props.handleTypes = cudaMemHandleTypeNone;
      props.location.type = cudaMemLocationTypeDevice;
      props.location.id = dev;
      SILE_CUDA_TRY(cudaMemPoolCreate(&g_pools[dev], &props));
      uint64_t keep = UINT64_MAX;
      SILE_CUDA_TRY(cudaMemPoolSetAttribute(g_pools[dev], cudaMemPoolAttrReleaseThreshold, &keep));
    }
    pool = g_pools[dev];
  }
  cudaError_t e = cudaMallocFromPoolAsync(ptr, bytes, pool, stream);
  if (e != cudaSuccess) return fail(SILE_ERR_CUDA, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
  return SILE_OK;
}

int device_work_counter(int** out) {
  int dev = 0;
  SILE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SILE_ERR_INVALID, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_work_counters[dev]) {
    int* p = nullptr;
    SILE_CUDA_TRY(cudaMalloc(&p, kWorkCounters * sizeof(int)));
    SILE_CUDA_TRY(cudaMemset(p, 0, kWorkCounters * sizeof(int)));
    g_work_counters[dev] = p;
  }
  *out = g_work_counters[dev] + (g_work_counter_next[dev]++ % kWorkCounters);
  return SILE_OK;
}

void note_kernel(const char* name, unsigned grid, unsigned block, size_t smem_bytes) {
  snprintf(t_last_kernel, sizeof(t_last_kernel), "%s grid=%u block=%u smem=%zu", name, grid, block, smem_bytes);
  static const bool print = std::getenv("SILE_PRINT_SOURCE") || std::getenv("SILE_PRINT_LLVMIR") || std::getenv("SILE_PRINT_TILEIR");
  if (print) fprintf(stderr, "[sile_cuda] launch %s\n", t_last_kernel);
}

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    else
      cudaGetLastError();
  });
  if (!g_encode_tiled) return fail(SILE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (uint32_t i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult r = g_encode_tiled(map, dtype, rank, const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(SILE_ERR_INVALID, "cuTensorMapEncodeTiled failed (%d): base %p dims [%llu,%llu] stride %llu box [%u,%u]",
                static_cast<int>(r), base, static_cast<unsigned long long>(dims[0]),
                static_cast<unsigned long long>(rank > 1 ? dims[1] : 0),
                static_cast<unsigned long long>(rank > 1 ? strides_bytes[0] : 0), box[0], rank > 1 ? box[1] : 0);
  return SILE_OK;
}

namespace {

size_t dtype_size(int dt) { return dt == SILE_DTYPE_F32 ? 4 : 2; }

int64_t grid_product(const uint32_t grid[3]) {
  return static_cast<int64_t>(grid[0]) * static_cast<int64_t>(grid[1]) * static_cast<int64_t>(grid[2]);
}

int64_t const_or_one(const SileKernelDesc* d, int i) { return d->consts[i] > 0 ? d->consts[i] : 1; }

// Buffers of a launch as (pointer, element count, element size, is_output).
struct ArgSpan {
  size_t bytes;
  bool is_input;
  bool is_output;
};

// Attention over the reference's f32 rank-2 tensors: shapes q [BH*S, D], kt [BH*D, S], v, o [BH*S, D].
struct AttnF32Dims {
  int64_t bh, s, d, rows, rows_written;
};
int attention_f32_dims(const SileKernelDesc* d, const int64_t* shapes, int64_t ns, int64_t ntg, AttnF32Dims* out) {
  if (ns != 8) return fail(SILE_ERR_INVALID, "attention (f32): expected q[BH*S,D] kt[BH*D,S] v[BH*S,D] o[BH*S,D]");
  const int64_t rows = shapes[0], dd = shapes[1], s = shapes[3];
  if (rows <= 0 || dd <= 0 || s <= 0) return fail(SILE_ERR_INVALID, "attention: non-positive dimension");
  if (rows % s != 0 || shapes[2] != rows / s * dd || shapes[4] != rows || shapes[5] != dd || shapes[6] != rows || shapes[7] != dd)
    return fail(SILE_ERR_INVALID, "attention (f32): inconsistent shapes q[%lld,%lld] kt[%lld,%lld] v[%lld,%lld] o[%lld,%lld]",
                (long long)shapes[0], (long long)shapes[1], (long long)shapes[2], (long long)shapes[3], (long long)shapes[4],
                (long long)shapes[5], (long long)shapes[6], (long long)shapes[7]);
  if (d->out_dtype != SILE_DTYPE_F32) return fail(SILE_ERR_UNSUPPORTED, "attention: f32 inputs give an f32 output");
  // [BM, D] query tiles and [D, BN] key tiles of the flattened tensors: a query tile must not
  // straddle two heads, and keys past the last whole BN tile would be dropped by the composed
  // kernel's loop (as the matmul's K remainder is) -- refused rather than silently different.
  const int64_t bm = d->consts[0] > 0 ? d->consts[0] : 1, bn = d->consts[1] > 0 ? d->consts[1] : 1;
  if (s % bm != 0 || s % bn != 0)
    return fail(SILE_ERR_UNSUPPORTED, "attention (f32): sequence length %lld must be a multiple of BM = %lld and BN = %lld", (long long)s,
                (long long)bm, (long long)bn);
  out->bh = rows / s;
  out->s = s;
  out->d = dd;
  out->rows = rows;
  out->rows_written = std::min<int64_t>(ntg < 0 ? 0 : ntg, rows / bm) * bm;  // q tiles [0, grid) run (cpu/codegen.rs:517-533)
  return SILE_OK;
}

// Validates shapes for `desc` and lists the byte size / direction of every buffer.
int describe_args(const SileKernelDesc* d, const int64_t* shapes, int64_t ns, int64_t ntg, std::vector<ArgSpan>* out) {
  out->clear();
  const size_t in_sz = dtype_size(d->in_dtype), out_sz = dtype_size(d->out_dtype);
  auto pos = [&](int64_t v) { return v > 0; };
  switch (d->op) {
    case SILE_OP_MATMUL: {
      if (ns != 6) return fail(SILE_ERR_INVALID, "matmul: expected 6 shape entries (a[M,K] b[K,N] c[M,N]), got %lld", (long long)ns);
      const int64_t m = shapes[0], k = shapes[1], n = shapes[5];
      if (!pos(m) || !pos(k) || !pos(n)) return fail(SILE_ERR_INVALID, "matmul: non-positive dimension");
      if (shapes[2] != k || shapes[3] != n || shapes[4] != m)
        return fail(SILE_ERR_INVALID, "matmul: inconsistent shapes a[%lld,%lld] b[%lld,%lld] c[%lld,%lld]", (long long)shapes[0],
                    (long long)shapes[1], (long long)shapes[2], (long long)shapes[3], (long long)shapes[4], (long long)shapes[5]);
      out->push_back({static_cast<size_t>(m * k) * in_sz, true, false});
      out->push_back({static_cast<size_t>(k * n) * in_sz, true, false});
      // C travels to the device only when part of it will not be written (ragged logical
      // tiles or a short grid): untouched elements must survive the round trip.
      const int64_t bm = const_or_one(d, 0), bn = const_or_one(d, 1);
      const bool partial = (m % bm) || (n % bn) || (ntg < (m / bm) * (n / bn));
      const bool seeded = (d->flags & SILE_FLAG_ACCUMULATE) != 0;  // C is read: D = C + A * B
      out->push_back({static_cast<size_t>(m * n) * out_sz, partial || seeded, true});
      return SILE_OK;
    }
    case SILE_OP_ATTENTION: {
      if (d->in_dtype == SILE_DTYPE_F32) {
        // The reference's own tensor model: f32, rank 2, K given transposed (its DSL has no
        // transpose op): q [BH*S, D], kt [BH*D, S], v [BH*S, D], o [BH*S, D].
        AttnF32Dims a;
        if (int rc = attention_f32_dims(d, shapes, ns, ntg, &a)) return rc;
        const size_t bytes = static_cast<size_t>(a.rows) * a.d * 4;
        out->push_back({bytes, true, false});
        out->push_back({bytes, true, false});
        out->push_back({bytes, true, false});
        out->push_back({bytes, a.rows_written < a.rows, true});  // untouched rows must survive the round trip
        return SILE_OK;
      }
      if (ns % 4 != 0 || ns / 4 < 2 || ns / 4 > 4) return fail(SILE_ERR_INVALID, "attention: expected 4 buffers of rank 2..4");
      const int64_t r = ns / 4;
      int64_t elems = 1;
      for (int64_t i = 0; i < r; ++i) {
        if (!pos(shapes[i])) return fail(SILE_ERR_INVALID, "attention: non-positive dimension");
        elems *= shapes[i];
      }
      for (int64_t a = 1; a < 4; ++a)
        for (int64_t i = 0; i < r; ++i)
          if (shapes[a * r + i] != shapes[i]) return fail(SILE_ERR_INVALID, "attention: q, k, v, o must share one shape");
      for (int a = 0; a < 3; ++a) out->push_back({static_cast<size_t>(elems) * in_sz, true, false});
      out->push_back({static_cast<size_t>(elems) * out_sz, false, true});
      return SILE_OK;
    }
    case SILE_OP_VEC_ADD: {
      if (ns != 3) return fail(SILE_ERR_INVALID, "vec_add: expected 3 rank-1 buffers");
      if (!pos(shapes[0]) || shapes[1] != shapes[0] || shapes[2] != shapes[0]) return fail(SILE_ERR_INVALID, "vec_add: lengths differ");
      out->push_back({static_cast<size_t>(shapes[0]) * 4, true, false});
      out->push_back({static_cast<size_t>(shapes[0]) * 4, true, false});
      out->push_back({static_cast<size_t>(shapes[0]) * 4, true, true});
      return SILE_OK;
    }
    case SILE_OP_RELU: {
      if (ns != 1 || !pos(shapes[0])) return fail(SILE_ERR_INVALID, "relu: expected one rank-1 buffer");
      out->push_back({static_cast<size_t>(shapes[0]) * 4, true, true});
      return SILE_OK;
    }
    case SILE_OP_SOFTMAX: {
      if (ns != 4) return fail(SILE_ERR_INVALID, "softmax: expected x[R,C] y[R,C]");
      if (!pos(shapes[0]) || !pos(shapes[1]) || shapes[2] != shapes[0] || shapes[3] != shapes[1])
        return fail(SILE_ERR_INVALID, "softmax: x and y shapes differ");
      out->push_back({static_cast<size_t>(shapes[0] * shapes[1]) * 4, true, false});
      out->push_back({static_cast<size_t>(shapes[0] * shapes[1]) * 4, true, true});
      return SILE_OK;
    }
    case SILE_OP_PARALLEL_REDUCE: {
      if (ns != 2 || !pos(shapes[0]) || shapes[1] != 1) return fail(SILE_ERR_INVALID, "parallel_reduce: expected a[N] out[1]");
      out->push_back({static_cast<size_t>(shapes[0]) * 4, true, false});
      out->push_back({4, true, true});  // atomic_add accumulates onto the caller's value
      return SILE_OK;
    }
    case SILE_OP_MATVEC: {
      if (ns != 4) return fail(SILE_ERR_INVALID, "matvec: expected x[M,K] y[K] z[M]");
      if (!pos(shapes[0]) || !pos(shapes[1]) || shapes[2] != shapes[1] || shapes[3] != shapes[0])
        return fail(SILE_ERR_INVALID, "matvec: inconsistent shapes");
      out->push_back({static_cast<size_t>(shapes[0] * shapes[1]) * 4, true, false});
      out->push_back({static_cast<size_t>(shapes[1]) * 4, true, false});
      out->push_back({static_cast<size_t>(shapes[0]) * 4, true, true});
      return SILE_OK;
    }
    default:
      return fail(SILE_ERR_UNSUPPORTED, "backend not implemented for op %d", d->op);
  }
}

int launch_device(const SileKernelDesc* d, void* const* buf, const int64_t* shapes, int64_t ns, int64_t ntg, cudaStream_t stream) {
  const bool f32_only = d->in_dtype == SILE_DTYPE_F32 && d->out_dtype == SILE_DTYPE_F32;
  switch (d->op) {
    case SILE_OP_MATMUL: {
      GemmProblem p;
      p.a = buf[0]; p.b = buf[1]; p.c = buf[2];
      p.m = shapes[0]; p.k = shapes[1]; p.n = shapes[5];
      p.in_dtype = d->in_dtype; p.out_dtype = d->out_dtype; p.b_layout = d->b_layout;
      p.bm = const_or_one(d, 0); p.bn = const_or_one(d, 1); p.bk = const_or_one(d, 2);
      p.num_threadgroups = ntg;
      p.accumulate = (d->flags & SILE_FLAG_ACCUMULATE) != 0;
      const size_t ws = gemm_workspace_bytes(p);
      void* wsp = nullptr;
      if (ws) {
        if (int rc = pool_alloc(&wsp, ws, stream)) return rc;
        p.workspace = wsp;
        p.workspace_bytes = ws;
      }
      const int rc = gemm_launch(p, stream);
      if (wsp) {
        cudaError_t e = cudaFreeAsync(wsp, stream);
        if (rc == SILE_OK && e != cudaSuccess) return fail(SILE_ERR_CUDA, "cudaFreeAsync failed: %s", cudaGetErrorString(e));
      }
      return rc;
    }
    case SILE_OP_ATTENTION: {
      if (d->in_dtype == SILE_DTYPE_F32) {
        // f32 rank-2 tensors with K transposed: convert to the [BH, S, D] bf16 layout of the
        // tensor-core kernel in scratch, run it on the heads the grid reaches, convert O back.
        AttnF32Dims a;
        if (int rc = attention_f32_dims(d, shapes, ns, ntg, &a)) return rc;
        if (a.rows_written == 0) return SILE_OK;
        const int64_t heads = (a.rows_written + a.s - 1) / a.s;
        const size_t plane = static_cast<size_t>(heads) * a.s * a.d * 2;
        void* ws = nullptr;
        if (int rc = pool_alloc(&ws, 4 * plane, stream)) return rc;
        char* qb = static_cast<char*>(ws);
        char *kb = qb + plane, *vb = kb + plane, *ob = vb + plane;
        const int64_t n = heads * a.s * a.d;
        int rc = cast_f32_to_bf16_launch(static_cast<const float*>(buf[0]), qb, n, stream);
        if (rc == SILE_OK) rc = transpose_cast_kt_launch(static_cast<const float*>(buf[1]), kb, heads, a.s, a.d, stream);
        if (rc == SILE_OK) rc = cast_f32_to_bf16_launch(static_cast<const float*>(buf[2]), vb, n, stream);
        if (rc == SILE_OK) {
          AttnProblem p;
          p.q = qb; p.k = kb; p.v = vb; p.o = ob;
          p.bh = heads; p.s = a.s; p.d = a.d;
          p.scale = d->scale;
          p.causal = d->causal;
          rc = attention_launch(p, stream);
        }
        if (rc == SILE_OK) rc = cast_bf16_to_f32_launch(ob, static_cast<float*>(buf[3]), a.rows_written * a.d, stream);
        cudaError_t e = cudaFreeAsync(ws, stream);
        if (rc == SILE_OK && e != cudaSuccess) return fail(SILE_ERR_CUDA, "cudaFreeAsync failed: %s", cudaGetErrorString(e));
        return rc;
      }
      const int64_t r = ns / 4;
      AttnProblem p;
      p.q = buf[0]; p.k = buf[1]; p.v = buf[2]; p.o = buf[3];
      p.d = shapes[r - 1];
      p.s = shapes[r - 2];
      p.bh = 1;
      for (int64_t i = 0; i + 2 < r; ++i) p.bh *= shapes[i];
      p.scale = d->scale;
      p.causal = d->causal;
      if (d->in_dtype != SILE_DTYPE_BF16 || d->out_dtype != SILE_DTYPE_BF16)
        return fail(SILE_ERR_UNSUPPORTED, "attention: bf16 in / bf16 out only");
      return attention_launch(p, stream);
    }
    case SILE_OP_VEC_ADD: {
      if (!f32_only) return fail(SILE_ERR_UNSUPPORTED, "vec_add: f32 only");
      // Tiles [0, grid) of TILE elements each are computed (cpu/codegen.rs:517-533).
      const int64_t tile = const_or_one(d, 0);
      const int64_t n = std::min<int64_t>(shapes[0] / tile, ntg) * tile;
      return vec_add_launch(static_cast<const float*>(buf[0]), static_cast<const float*>(buf[1]), static_cast<float*>(buf[2]), n, stream);
    }
    case SILE_OP_RELU: {
      if (!f32_only) return fail(SILE_ERR_UNSUPPORTED, "relu: f32 only");
      if (ntg < 1) return SILE_OK;
      return relu_launch(static_cast<float*>(buf[0]), shapes[0], stream);
    }
    case SILE_OP_SOFTMAX: {
      if (!f32_only) return fail(SILE_ERR_UNSUPPORTED, "softmax: f32 only");
      const int64_t rows = shapes[2], cols = shapes[3];
      const int64_t bm = const_or_one(d, 0);
      const int64_t bn = d->consts[1] > 0 ? d->consts[1] : cols;
      if (bn > cols) return SILE_OK;  // no whole tile fits the row: nothing is launched
      if (bn != cols) {
        // BN narrower than the row: every [BM, BN] tile is a softmax of its own, as in the
        // reference (examples/softmax.rs:3-16); columns past the last whole tile stay untouched
        const int64_t tiles_n = cols / bn;
        const int64_t num_tiles = std::min<int64_t>(ntg, (rows / bm) * tiles_n);
        return softmax_tiles_launch(static_cast<const float*>(buf[0]), shapes[1], static_cast<float*>(buf[1]), cols, rows / bm * bm,
                                    tiles_n, bm, bn, num_tiles, stream);
      }
      const int64_t r = std::min<int64_t>(rows / bm, ntg) * bm;
      return softmax_rows_launch(static_cast<const float*>(buf[0]), shapes[1], static_cast<float*>(buf[1]), cols, r, cols, stream);
    }
    case SILE_OP_PARALLEL_REDUCE: {
      if (!f32_only) return fail(SILE_ERR_UNSUPPORTED, "parallel_reduce: f32 only");
      const int64_t tile = const_or_one(d, 0);
      const int64_t n = std::min<int64_t>(shapes[0] / tile, ntg) * tile;
      return reduce_sum_launch(static_cast<const float*>(buf[0]), n, static_cast<float*>(buf[1]), stream);
    }
    case SILE_OP_MATVEC: {
      if (!f32_only) return fail(SILE_ERR_UNSUPPORTED, "matvec: f32 only");
      const int64_t bm = const_or_one(d, 0), bk = const_or_one(d, 1);
      const int64_t m = std::min<int64_t>(shapes[0] / bm, ntg) * bm;
      const int64_t k = shapes[1] / bk * bk;
      if (k != shapes[1]) return fail(SILE_ERR_UNSUPPORTED, "matvec: K must be a multiple of BK");
      return matvec_launch(static_cast<const float*>(buf[0]), static_cast<const float*>(buf[1]), static_cast<float*>(buf[2]), m, shapes[1], stream);
    }
    default:
      return fail(SILE_ERR_UNSUPPORTED, "backend not implemented for op %d", d->op);
  }
}

int validate_desc(const SileKernelDesc* d) {
  if (!d) return fail(SILE_ERR_INVALID, "null kernel description");
  if (d->struct_size != sizeof(SileKernelDesc))
    return fail(SILE_ERR_INVALID, "SileKernelDesc size %u does not match this library (%zu)", d->struct_size, sizeof(SileKernelDesc));
  return SILE_OK;
}

// Reads and clears both per-device status words: the one every ordinary launch reports to and
// the one inside the library image that the allocation-free matmul uses.  Either may hold a
// time-out from an earlier asynchronous launch; the first one found is reported.
int read_and_clear_status() {
  int* word = nullptr;
  if (int rc = device_status_word(&word)) return rc;
  int v = 0;
  SILE_CUDA_TRY(cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) SILE_CUDA_TRY(cudaMemset(word, 0, sizeof(int)));
  int v2 = 0;
  if (int rc = noalloc_read_and_clear_status(&v2)) return rc;
  return decode_status_word(v != 0 ? v : v2);
}

// Large 16-bit matmuls from host memory: A travels in row chunks on one stream, each chunk's
// GEMM runs on a second as soon as its rows (and all of B) have arrived, and its rows of C return
// on a third, so the two PCIe directions and the tensor cores work at the same time.  Only for
// launches that write every element of C (whole logical tiles, full grid), where chunking the
// rows cannot change which elements are written.
// The three streams (copies in, kernels, copies out) and the events of the host-buffer pipelines,
// made once per host thread and device and reused by later calls.
struct PipelineStreams {
  int device = -1;
  cudaStream_t in = nullptr, run = nullptr, out = nullptr;
  std::vector<cudaEvent_t> events;
};
int pipeline_streams(PipelineStreams** out) {
  static thread_local PipelineStreams cached;
  int dev_now = 0;
  SILE_CUDA_TRY(cudaGetDevice(&dev_now));
  if (cached.device != dev_now) {
    cached = PipelineStreams{};  // (streams and events of a previously used device are left to that device)
    SILE_CUDA_TRY(cudaStreamCreateWithFlags(&cached.in, cudaStreamNonBlocking));
    SILE_CUDA_TRY(cudaStreamCreateWithFlags(&cached.run, cudaStreamNonBlocking));
    SILE_CUDA_TRY(cudaStreamCreateWithFlags(&cached.out, cudaStreamNonBlocking));
    cached.device = dev_now;
  }
  *out = &cached;
  return SILE_OK;
}

// Host-buffer attention over many heads: heads are independent, so q, k, v travel in chunks of
// heads, each chunk's kernel starts when its copies have arrived and its o leaves while later
// chunks are still arriving.  The step is then bounded by the host link (three inputs in, one
// output back, full duplex) instead of being the sum of copies and kernel.
int launch_host_attention_pipelined(const SileKernelDesc* d, void* const* host, const int64_t* shapes, int64_t ns, bool* handled) {
  *handled = false;
  if (d->in_dtype != SILE_DTYPE_BF16 || d->out_dtype != SILE_DTYPE_BF16) return SILE_OK;
  const int64_t r = ns / 4;
  if (ns % 4 != 0 || r < 3 || r > 4) return SILE_OK;
  const int64_t dd = shapes[r - 1], sq = shapes[r - 2];
  int64_t bh = 1;
  for (int64_t i = 0; i + 2 < r; ++i) bh *= shapes[i];
  const size_t head_bytes = static_cast<size_t>(sq) * dd * 2;
  // chunks of about 8 MiB per tensor, at least 4 chunks; small problems take the plain path
  const int64_t heads_per_chunk = std::max<int64_t>(1, static_cast<int64_t>((size_t(8) << 20) / std::max<size_t>(head_bytes, 1)));
  if (dd != 128 || bh < 4 * heads_per_chunk || head_bytes * bh < (size_t(64) << 20)) return SILE_OK;
  *handled = true;
  PipelineStreams* streams = nullptr;
  if (int prc = pipeline_streams(&streams)) return prc;
  PipelineStreams& cached = *streams;
  void* dev[4] = {nullptr, nullptr, nullptr, nullptr};
  size_t events_used = 0;
  int rc = SILE_OK;
  auto check = [&](cudaError_t e, const char* what) {
    if (e != cudaSuccess && rc == SILE_OK) rc = fail(SILE_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
    return e == cudaSuccess;
  };
  auto new_event = [&]() {
    if (events_used == cached.events.size()) {
      cudaEvent_t ev = nullptr;
      check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
      cached.events.push_back(ev);
    }
    return cached.events[events_used++];
  };
  for (int i = 0; i < 4 && rc == SILE_OK; ++i) rc = pool_alloc(&dev[i], head_bytes * bh, cached.in);
  for (int64_t h0 = 0; h0 < bh && rc == SILE_OK; h0 += heads_per_chunk) {
    const int64_t heads = std::min(heads_per_chunk, bh - h0);
    const size_t off = head_bytes * h0, bytes = head_bytes * heads;
    for (int i = 0; i < 3; ++i)
      check(cudaMemcpyAsync(static_cast<char*>(dev[i]) + off, static_cast<const char*>(host[i]) + off, bytes, cudaMemcpyHostToDevice, cached.in),
            "host->device copy");
    cudaEvent_t arrived = new_event();
    check(cudaEventRecord(arrived, cached.in), "cudaEventRecord");
    check(cudaStreamWaitEvent(cached.run, arrived, 0), "cudaStreamWaitEvent");
    if (rc != SILE_OK) break;
    AttnProblem p;
    p.q = static_cast<char*>(dev[0]) + off; p.k = static_cast<char*>(dev[1]) + off; p.v = static_cast<char*>(dev[2]) + off;
    p.o = static_cast<char*>(dev[3]) + off;
    p.bh = heads; p.s = sq; p.d = dd;
    p.scale = d->scale;
    p.causal = d->causal;
    rc = attention_launch(p, cached.run);
    if (rc != SILE_OK) break;
    cudaEvent_t computed = new_event();
    check(cudaEventRecord(computed, cached.run), "cudaEventRecord");
    check(cudaStreamWaitEvent(cached.out, computed, 0), "cudaStreamWaitEvent");
    check(cudaMemcpyAsync(static_cast<char*>(host[3]) + off, static_cast<char*>(dev[3]) + off, bytes, cudaMemcpyDeviceToHost, cached.out),
          "device->host copy");
  }
  check(cudaStreamSynchronize(cached.in), "host->device copy");
  check(cudaStreamSynchronize(cached.run), "kernel execution");
  check(cudaStreamSynchronize(cached.out), "device->host copy");
  if (rc == SILE_OK) rc = read_and_clear_status();
  for (void* ptr : dev)
    if (ptr) cudaFreeAsync(ptr, cached.in);
  cudaStreamSynchronize(cached.in);
  return rc;
}

int launch_host_matmul_pipelined(const SileKernelDesc* d, void* const* host, const int64_t* shapes, bool* handled) {
  *handled = false;
  const int64_t m = shapes[0], k = shapes[1], n = shapes[5];
  const int64_t bm = const_or_one(d, 0);
  if (d->in_dtype == SILE_DTYPE_F32 || d->b_layout != SILE_LAYOUT_COL_MAJOR) return SILE_OK;
  // Rows per chunk: small chunks shorten the pipeline's fill and drain, large ones keep the GEMM
  // efficient.  SILE_CUDA_HOST_CHUNK_ROWS overrides the default for tuning.
  int64_t base_rows = 1024;
  if (const char* env = std::getenv("SILE_CUDA_HOST_CHUNK_ROWS")) {
    const long v = std::atol(env);
    if (v >= 128 && v % 128 == 0) base_rows = v;
  }
  int64_t rows = base_rows;
  while (rows % bm != 0 && rows < m) rows += base_rows;   // chunk boundaries must fall on logical tile boundaries
  if (m < 4 * rows || rows % bm != 0 || m % bm != 0 || static_cast<double>(m) * n * k < 1e11) return SILE_OK;
  *handled = true;
  const size_t in_sz = dtype_size(d->in_dtype), out_sz = dtype_size(d->out_dtype);
  PipelineStreams* streams = nullptr;
  if (int prc = pipeline_streams(&streams)) return prc;
  PipelineStreams& cached = *streams;
  cudaStream_t s_in = cached.in, s_run = cached.run, s_out = cached.out;
  // Row chunks: full ones, then the last one halved down to 256 rows, so that what is left to do
  // after the last input row has arrived (one GEMM and one copy back) is small.
  std::vector<int64_t> chunk_rows;
  {
    int64_t left = m;
    while (left > rows) {
      chunk_rows.push_back(rows);
      left -= rows;
    }
    while (left >= 512 && (left / 2) % bm == 0 && (left / 2) % 128 == 0) {
      chunk_rows.push_back(left / 2);
      left -= left / 2;
    }
    chunk_rows.push_back(left);
  }
  void *da = nullptr, *db = nullptr, *dc = nullptr;
  size_t events_used = 0;
  int rc = SILE_OK;
  auto check = [&](cudaError_t e, const char* what) {
    if (e != cudaSuccess && rc == SILE_OK) rc = fail(SILE_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
    return e == cudaSuccess;
  };
  auto new_event = [&]() {
    if (events_used == cached.events.size()) {
      cudaEvent_t ev = nullptr;
      check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
      cached.events.push_back(ev);
    }
    return cached.events[events_used++];
  };
  if (rc == SILE_OK) rc = pool_alloc(&da, static_cast<size_t>(m * k) * in_sz, s_in);
  if (rc == SILE_OK) rc = pool_alloc(&db, static_cast<size_t>(k * n) * in_sz, s_in);
  if (rc == SILE_OK) rc = pool_alloc(&dc, static_cast<size_t>(m * n) * out_sz, s_in);
  if (rc == SILE_OK) {
    check(cudaMemcpyAsync(db, host[1], static_cast<size_t>(k * n) * in_sz, cudaMemcpyHostToDevice, s_in), "host->device copy");
    int64_t r0 = 0;
    for (size_t ci = 0; ci < chunk_rows.size() && rc == SILE_OK; r0 += chunk_rows[ci], ++ci) {
      const int64_t rc_rows = chunk_rows[ci];
      const size_t a_off = static_cast<size_t>(r0 * k) * in_sz, c_off = static_cast<size_t>(r0 * n) * out_sz;
      check(cudaMemcpyAsync(static_cast<char*>(da) + a_off, static_cast<const char*>(host[0]) + a_off,
                            static_cast<size_t>(rc_rows * k) * in_sz, cudaMemcpyHostToDevice, s_in), "host->device copy");
      cudaEvent_t arrived = new_event();
      check(cudaEventRecord(arrived, s_in), "cudaEventRecord");
      check(cudaStreamWaitEvent(s_run, arrived, 0), "cudaStreamWaitEvent");
      if (rc != SILE_OK) break;
      GemmProblem p;
      p.a = static_cast<char*>(da) + a_off; p.b = db; p.c = static_cast<char*>(dc) + c_off;
      p.m = rc_rows; p.n = n; p.k = k;
      p.in_dtype = d->in_dtype; p.out_dtype = d->out_dtype; p.b_layout = d->b_layout;
      p.bm = bm; p.bn = const_or_one(d, 1); p.bk = const_or_one(d, 2);
      rc = gemm_launch(p, s_run);
      if (rc != SILE_OK) break;
      cudaEvent_t computed = new_event();
      check(cudaEventRecord(computed, s_run), "cudaEventRecord");
      check(cudaStreamWaitEvent(s_out, computed, 0), "cudaStreamWaitEvent");
      check(cudaMemcpyAsync(static_cast<char*>(host[2]) + c_off, static_cast<char*>(dc) + c_off,
                            static_cast<size_t>(rc_rows * n) * out_sz, cudaMemcpyDeviceToHost, s_out), "device->host copy");
    }
  }
  check(cudaStreamSynchronize(s_in), "host->device copy");
  check(cudaStreamSynchronize(s_run), "kernel execution");
  check(cudaStreamSynchronize(s_out), "device->host copy");
  if (rc == SILE_OK) rc = read_and_clear_status();
  for (void* ptr : {da, db, dc})
    if (ptr) cudaFreeAsync(ptr, s_in);
  cudaStreamSynchronize(s_in);
  return rc;
}

int launch_host(const SileKernelDesc* d, void* const* host, const int64_t* shapes, int64_t ns, int64_t ntg) {
  if (int rc = validate_desc(d)) return rc;
  if (int rc = check_device()) return rc;
  if (!host || !shapes) return fail(SILE_ERR_INVALID, "null argument");
  std::vector<ArgSpan> args;
  if (int rc = describe_args(d, shapes, ns, ntg, &args)) return rc;
  if (d->op == SILE_OP_ATTENTION && host[0] && host[1] && host[2] && host[3]) {
    bool handled = false;
    const int rc = launch_host_attention_pipelined(d, host, shapes, ns, &handled);
    if (handled) {
      if (rc == SILE_OK) t_last_status = SILE_OK;
      return rc;
    }
  }
  if (d->op == SILE_OP_MATMUL && !args[2].is_input && host[0] && host[1] && host[2]) {
    bool handled = false;
    const int rc = launch_host_matmul_pipelined(d, host, shapes, &handled);
    if (handled) {
      if (rc == SILE_OK) t_last_status = SILE_OK;
      return rc;
    }
  }
  cudaStream_t stream = nullptr;
  SILE_CUDA_TRY(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  std::vector<void*> dev(args.size(), nullptr);
  int rc = SILE_OK;
  auto cleanup = [&]() {
    for (void* p : dev)
      if (p) cudaFreeAsync(p, stream);
    cudaStreamSynchronize(stream);
    cudaStreamDestroy(stream);
  };
  for (size_t i = 0; i < args.size() && rc == SILE_OK; ++i) {
    if (!host[i]) { rc = fail(SILE_ERR_INVALID, "null buffer %zu", i); break; }
    rc = pool_alloc(&dev[i], std::max<size_t>(args[i].bytes, 16), stream);
    if (rc != SILE_OK) break;
    if (args[i].is_input) {
      cudaError_t e = cudaMemcpyAsync(dev[i], host[i], args[i].bytes, cudaMemcpyHostToDevice, stream);
      if (e != cudaSuccess) rc = fail(SILE_ERR_CUDA, "host->device copy failed: %s", cudaGetErrorString(e));
    }
  }
  if (rc == SILE_OK) rc = launch_device(d, dev.data(), shapes, ns, ntg, stream);
  if (rc == SILE_OK) {
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) rc = fail(SILE_ERR_CUDA, "kernel execution failed: %s", cudaGetErrorString(e));
  }
  if (rc == SILE_OK) rc = read_and_clear_status();
  for (size_t i = 0; i < args.size() && rc == SILE_OK; ++i) {
    if (args[i].is_output) {
      cudaError_t e = cudaMemcpyAsync(host[i], dev[i], args[i].bytes, cudaMemcpyDeviceToHost, stream);
      if (e != cudaSuccess) rc = fail(SILE_ERR_CUDA, "device->host copy failed: %s", cudaGetErrorString(e));
    }
  }
  if (rc == SILE_OK) {
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) rc = fail(SILE_ERR_CUDA, "device->host copy failed: %s", cudaGetErrorString(e));
  }
  cleanup();
  if (rc == SILE_OK) t_last_status = SILE_OK;
  return rc;
}

SileKernelDesc f32_desc(int op) {
  SileKernelDesc d;
  std::memset(&d, 0, sizeof(d));
  d.struct_size = sizeof(d);
  d.op = op;
  d.in_dtype = SILE_DTYPE_F32;
  d.out_dtype = SILE_DTYPE_F32;
  d.b_layout = SILE_LAYOUT_ROW_MAJOR;
  d.scale = 1.0f;
  return d;
}

}  // namespace
}  // namespace sile

using namespace sile;

extern "C" {

int sile_cuda_version(void) { return 100; }

int sile_cuda_gemm_slice_plan(int32_t tiles, int32_t cta_pairs, int32_t destinations, int32_t exchange_bound, char* out, int64_t capacity) {
  return gemm_slice_plan_text(tiles, cta_pairs, destinations, exchange_bound, out, capacity > 0 ? static_cast<size_t>(capacity) : 0);
}

const char* sile_cuda_last_error(void) { return t_last_error.c_str(); }
const char* sile_cuda_last_kernel(void) { return t_last_kernel; }
int sile_cuda_last_status(void) { return t_last_status; }

int sile_cuda_decode_status(int status_word) { return decode_status_word(status_word); }

int sile_cuda_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int sile_cuda_set_device(int index) {
  int n = sile_cuda_device_count();
  if (index < 0 || index >= n) return fail(SILE_ERR_NO_DEVICE, "invalid device: cuda:%d (%d visible)", index, n);
  SILE_CUDA_TRY(cudaSetDevice(index));
  return check_device();
}

int sile_cuda_synchronize(void* stream) {
  if (int rc = check_device()) return rc;
  SILE_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return read_and_clear_status();
}

int sile_cuda_malloc(void** dev_ptr, size_t bytes) {
  if (!dev_ptr) return fail(SILE_ERR_INVALID, "null argument");
  *dev_ptr = nullptr;
  if (int rc = check_device()) return rc;
  if (bytes == 0) return SILE_OK;
  SILE_CUDA_TRY(cudaMalloc(dev_ptr, bytes));
  return SILE_OK;
}

int sile_cuda_free(void* dev_ptr) {
  if (!dev_ptr) return SILE_OK;
  SILE_CUDA_TRY(cudaFree(dev_ptr));
  return SILE_OK;
}

int sile_cuda_memcpy_h2d(void* dev_dst, const void* host_src, size_t bytes, void* stream) {
  if (bytes == 0) return SILE_OK;
  if (!dev_dst || !host_src) return fail(SILE_ERR_INVALID, "null argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SILE_CUDA_TRY(cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, st));
  SILE_CUDA_TRY(cudaStreamSynchronize(st));
  return SILE_OK;
}

int sile_cuda_memcpy_d2h(void* host_dst, const void* dev_src, size_t bytes, void* stream) {
  if (bytes == 0) return SILE_OK;
  if (!host_dst || !dev_src) return fail(SILE_ERR_INVALID, "null argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SILE_CUDA_TRY(cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, st));
  SILE_CUDA_TRY(cudaStreamSynchronize(st));
  return read_and_clear_status();
}

int sile_cuda_memset(void* dev_dst, int byte_value, size_t bytes, void* stream) {
  if (bytes == 0) return SILE_OK;
  if (!dev_dst) return fail(SILE_ERR_INVALID, "null argument");
  SILE_CUDA_TRY(cudaMemsetAsync(dev_dst, byte_value, bytes, static_cast<cudaStream_t>(stream)));
  return SILE_OK;
}

int sile_cuda_stream_create(void** stream) {
  if (!stream) return fail(SILE_ERR_INVALID, "null argument");
  *stream = nullptr;
  if (int rc = check_device()) return rc;
  cudaStream_t st = nullptr;
  SILE_CUDA_TRY(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  *stream = st;
  return SILE_OK;
}

int sile_cuda_stream_destroy(void* stream) {
  if (!stream) return SILE_OK;
  SILE_CUDA_TRY(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
  return SILE_OK;
}

size_t sile_cuda_matmul_workspace_bytes(int64_t m, int64_t n, int64_t k, int32_t in_dtype) {
  GemmProblem p;
  p.m = m; p.n = n; p.k = k; p.in_dtype = in_dtype;
  return gemm_workspace_bytes(p);
}

int sile_cuda_bind_consts(const char* name, const int64_t* consts, int64_t n) {
  if (!name || (!consts && n > 0)) return fail(SILE_ERR_INVALID, "null argument");
  auto set = [&](int64_t* dst, int64_t want) -> int {
    if (n != want) return fail(SILE_ERR_INVALID, "%s takes %lld const generics, got %lld", name, (long long)want, (long long)n);
    for (int64_t i = 0; i < want; ++i) {
      if (consts[i] <= 0) return fail(SILE_ERR_INVALID, "%s: const generic %lld must be positive", name, (long long)i);
      dst[i] = consts[i];
    }
    return SILE_OK;
  };
  if (!std::strcmp(name, "matmul") || !std::strcmp(name, "gemm")) return set(t_consts.matmul, 3);
  if (!std::strcmp(name, "matmul_acc")) return set(t_consts.matmul_acc, 3);
  if (!std::strcmp(name, "vec_add")) return set(t_consts.vec_add, 1);
  if (!std::strcmp(name, "softmax")) return set(t_consts.softmax, 2);
  if (!std::strcmp(name, "parallel_reduce")) return set(t_consts.parallel_reduce, 1);
  if (!std::strcmp(name, "matvec")) return set(t_consts.matvec, 2);
  if (!std::strcmp(name, "attention")) {
    // BM, BN and the causal flag (0 / 1), which is not a tile size and may be zero
    if (n != 3) return fail(SILE_ERR_INVALID, "attention takes 3 const generics (BM, BN, causal), got %lld", (long long)n);
    if (consts[0] <= 0 || consts[1] <= 0 || (consts[2] != 0 && consts[2] != 1))
      return fail(SILE_ERR_INVALID, "attention: BM and BN must be positive and causal 0 or 1");
    for (int i = 0; i < 3; ++i) t_consts.attention[i] = consts[i];
    return SILE_OK;
  }
  return fail(SILE_ERR_UNSUPPORTED, "no kernel named %s", name);
}

int sile_cuda_bind_scale(const char* name, float scale) {
  if (!name) return fail(SILE_ERR_INVALID, "null argument");
  if (std::strcmp(name, "attention") != 0) return fail(SILE_ERR_UNSUPPORTED, "kernel %s has no scale literal", name);
  if (!(scale > 0.0f)) return fail(SILE_ERR_INVALID, "attention: scale must be positive");
  t_consts.attention_scale = scale;
  return SILE_OK;
}

int sile_cuda_launch(const SileKernelDesc* desc, void* const* dev_buffers, const int64_t* shapes, int64_t num_shapes,
                     const uint32_t grid[3], void* stream) {
  if (int rc = validate_desc(desc)) return rc;
  if (int rc = check_device()) return rc;
  if (!dev_buffers || !shapes || !grid) return fail(SILE_ERR_INVALID, "null argument");
  std::vector<ArgSpan> args;
  if (int rc = describe_args(desc, shapes, num_shapes, grid_product(grid), &args)) return rc;
  for (size_t i = 0; i < args.size(); ++i)
    if (!dev_buffers[i]) return fail(SILE_ERR_INVALID, "null buffer %zu", i);
  const int rc = launch_device(desc, dev_buffers, shapes, num_shapes, grid_product(grid), static_cast<cudaStream_t>(stream));
  if (rc == SILE_OK) t_last_status = SILE_OK;
  return rc;
}

int sile_cuda_launch_host(const SileKernelDesc* desc, void* const* host_buffers, const int64_t* shapes, int64_t num_shapes,
                          const uint32_t grid[3]) {
  if (!grid) return fail(SILE_ERR_INVALID, "null argument");
  return launch_host(desc, host_buffers, shapes, num_shapes, grid_product(grid));
}

int sile_cuda_matmul_shard(const SileKernelDesc* desc, const void* a, const void* b_shard, void* c, int64_t m, int64_t n_total,
                           int64_t k, int64_t n_begin, int64_t n_count, void* stream) {
  if (int rc = validate_desc(desc)) return rc;
  if (int rc = check_device()) return rc;
  if (desc->op != SILE_OP_MATMUL) return fail(SILE_ERR_INVALID, "matmul_shard: description is not a matmul");
  if (!a || !b_shard || !c) return fail(SILE_ERR_INVALID, "null buffer");
  if (n_begin < 0 || n_count <= 0 || n_begin + n_count > n_total) return fail(SILE_ERR_INVALID, "matmul_shard: column block out of range");
  if (desc->flags & SILE_FLAG_ACCUMULATE) return fail(SILE_ERR_UNSUPPORTED, "matmul_shard: seeded accumulator not supported");
  if (desc->in_dtype == SILE_DTYPE_F32 || desc->b_layout != SILE_LAYOUT_COL_MAJOR)
    return fail(SILE_ERR_UNSUPPORTED, "matmul_shard: 16-bit operands with column-major B only (a column block of B must be contiguous)");
  GemmProblem p;
  p.a = a; p.b = b_shard;
  p.c = static_cast<char*>(c) + static_cast<size_t>(n_begin) * dtype_size(desc->out_dtype);
  p.m = m; p.n = n_count; p.k = k; p.ldc = n_total;
  p.in_dtype = desc->in_dtype; p.out_dtype = desc->out_dtype; p.b_layout = desc->b_layout;
  p.bm = const_or_one(desc, 0); p.bn = const_or_one(desc, 1); p.bk = const_or_one(desc, 2);
  const int rc = gemm_launch(p, static_cast<cudaStream_t>(stream));
  if (rc == SILE_OK) t_last_status = SILE_OK;
  return rc;
}

int sile_cuda_matmul_allgather(const SileKernelDesc* desc, const void* a, const void* b_shard, void* const* c_peers, int32_t world,
                               int32_t rank, int64_t m, int64_t n_total, int64_t k, void* stream) {
  if (int rc = validate_desc(desc)) return rc;
  if (int rc = check_device()) return rc;
  if (desc->op != SILE_OP_MATMUL) return fail(SILE_ERR_INVALID, "matmul_allgather: description is not a matmul");
  if (!a || !b_shard || !c_peers) return fail(SILE_ERR_INVALID, "null buffer");
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(SILE_ERR_INVALID, "matmul_allgather: bad rank %d of %d (at most 8)", rank, world);
  if (n_total % world != 0) return fail(SILE_ERR_INVALID, "matmul_allgather: N = %lld does not split into %d column blocks", (long long)n_total, world);
  if (desc->flags & SILE_FLAG_ACCUMULATE)
    return fail(SILE_ERR_UNSUPPORTED, "matmul_allgather: a seeded accumulator would be read from every rank's buffer; not supported");
  if (desc->in_dtype == SILE_DTYPE_F32 || desc->b_layout != SILE_LAYOUT_COL_MAJOR)
    return fail(SILE_ERR_UNSUPPORTED, "matmul_allgather: 16-bit operands with column-major B only");
  const int64_t n_count = n_total / world, n_begin = n_count * rank;
  GemmProblem p;
  p.a = a; p.b = b_shard;
  p.m = m; p.n = n_count; p.k = k; p.ldc = n_total;
  p.in_dtype = desc->in_dtype; p.out_dtype = desc->out_dtype; p.b_layout = desc->b_layout;
  p.bm = const_or_one(desc, 0); p.bn = const_or_one(desc, 1); p.bk = const_or_one(desc, 2);
  const size_t off = static_cast<size_t>(n_begin) * dtype_size(desc->out_dtype);
  for (int i = 0; i < world; ++i) {
    if (!c_peers[i]) return fail(SILE_ERR_INVALID, "matmul_allgather: null destination %d", i);
    p.peer_c[i] = static_cast<char*>(c_peers[i]) + off;
  }
  p.c = p.peer_c[rank];
  p.num_peers = world;
  p.peer_first = rank;
  const int rc = gemm_launch(p, static_cast<cudaStream_t>(stream));
  if (rc == SILE_OK) t_last_status = SILE_OK;
  return rc;
}

int sile_cuda_attention_allgather(const SileKernelDesc* desc, const void* q, const void* k, const void* v, void* const* o_peers,
                                  int32_t world, int32_t rank, int64_t bh_local, int64_t s, void* stream) {
  if (int rc = validate_desc(desc)) return rc;
  if (int rc = check_device()) return rc;
  if (desc->op != SILE_OP_ATTENTION) return fail(SILE_ERR_INVALID, "attention_allgather: description is not an attention");
  if (desc->in_dtype != SILE_DTYPE_BF16 || desc->out_dtype != SILE_DTYPE_BF16)
    return fail(SILE_ERR_UNSUPPORTED, "attention: bf16 in / bf16 out only");
  if (!o_peers) return fail(SILE_ERR_INVALID, "null buffer");
  if (world < 1 || world > 8 || rank < 0 || rank >= world)
    return fail(SILE_ERR_INVALID, "attention_allgather: bad rank %d of %d (at most 8)", rank, world);
  AttnProblem p;
  p.q = q; p.k = k; p.v = v;
  p.bh = bh_local; p.s = s; p.d = 128;
  p.scale = desc->scale;
  p.causal = desc->causal;
  p.num_peers = world;
  p.peer_first = rank;
  p.bh_total = bh_local * world;
  p.bh_offset = bh_local * rank;
  for (int i = 0; i < world; ++i) p.peer_o[i] = o_peers[i];
  const int rc = attention_launch(p, static_cast<cudaStream_t>(stream));
  if (rc == SILE_OK) t_last_status = SILE_OK;
  return rc;
}

int sile_cuda_unshard_columns(void* dst, const void* src, int64_t parts, int64_t rows, int64_t cols, int32_t dtype, void* stream) {
  if (int rc = check_device()) return rc;
  const int rc = unshard_columns_launch(dst, src, parts, rows, cols, static_cast<int>(dtype_size(dtype)), static_cast<cudaStream_t>(stream));
  if (rc == SILE_OK) t_last_status = SILE_OK;
  return rc;
}

void sile_kernel_matmul(void** buffers, int64_t num_threadgroups, int64_t threads_per_group, const int64_t* shapes, int64_t num_shapes) {
  SileKernelDesc d = f32_desc(SILE_OP_MATMUL);
  for (int i = 0; i < 3; ++i) d.consts[i] = t_consts.matmul[i];
  launch_host(&d, buffers, shapes, num_shapes, num_threadgroups * threads_per_group);
}
void sile_kernel_matmul_acc(void** buffers, int64_t num_threadgroups, int64_t threads_per_group, const int64_t* shapes, int64_t num_shapes) {
  SileKernelDesc d = f32_desc(SILE_OP_MATMUL);
  d.flags = SILE_FLAG_ACCUMULATE;
  for (int i = 0; i < 3; ++i) d.consts[i] = t_consts.matmul_acc[i];
  launch_host(&d, buffers, shapes, num_shapes, num_threadgroups * threads_per_group);
}
void sile_kernel_vec_add(void** buffers, int64_t num_threadgroups, int64_t threads_per_group, const int64_t* shapes, int64_t num_shapes) {
  SileKernelDesc d = f32_desc(SILE_OP_VEC_ADD);
  d.consts[0] = t_consts.vec_add[0];
  launch_host(&d, buffers, shapes, num_shapes, num_threadgroups * threads_per_group);
}
void sile_kernel_relu(void** buffers, int64_t num_threadgroups, int64_t threads_per_group, const int64_t* shapes, int64_t num_shapes) {
  SileKernelDesc d = f32_desc(SILE_OP_RELU);
  launch_host(&d, buffers, shapes, num_shapes, num_threadgroups * threads_per_group);
}
void sile_kernel_softmax(void** buffers, int64_t num_threadgroups, int64_t threads_per_group, const int64_t* shapes, int64_t num_shapes) {
  SileKernelDesc d = f32_desc(SILE_OP_SOFTMAX);
  d.consts[0] = t_consts.softmax[0];
  d.consts[1] = t_consts.softmax[1];
  launch_host(&d, buffers, shapes, num_shapes, num_threadgroups * threads_per_group);
}
void sile_kernel_parallel_reduce(void** buffers, int64_t num_threadgroups, int64_t threads_per_group, const int64_t* shapes, int64_t num_shapes) {
  SileKernelDesc d = f32_desc(SILE_OP_PARALLEL_REDUCE);
  d.consts[0] = t_consts.parallel_reduce[0];
  launch_host(&d, buffers, shapes, num_shapes, num_threadgroups * threads_per_group);
}
void sile_kernel_attention(void** buffers, int64_t num_threadgroups, int64_t threads_per_group, const int64_t* shapes, int64_t num_shapes) {
  SileKernelDesc d = f32_desc(SILE_OP_ATTENTION);
  d.consts[0] = t_consts.attention[0];
  d.consts[1] = t_consts.attention[1];
  d.causal = static_cast<int32_t>(t_consts.attention[2]);
  d.scale = t_consts.attention_scale;
  launch_host(&d, buffers, shapes, num_shapes, num_threadgroups * threads_per_group);
}
void sile_kernel_matvec(void** buffers, int64_t num_threadgroups, int64_t threads_per_group, const int64_t* shapes, int64_t num_shapes) {
  SileKernelDesc d = f32_desc(SILE_OP_MATVEC);
  d.consts[0] = t_consts.matvec[0];
  d.consts[1] = t_consts.matvec[1];
  launch_host(&d, buffers, shapes, num_shapes, num_threadgroups * threads_per_group);
}

}  // extern "C"
