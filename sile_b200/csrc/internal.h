// Declarations shared by the translation units of libsile_cuda.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/sile_cuda.h"

namespace sile {

// Records a message retrievable through sile_cuda_last_error() and returns `code`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

#define SILE_CUDA_TRY(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      return ::sile::fail(SILE_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                 \
                          cudaGetErrorString(_e), __FILE__, __LINE__);                   \
  } while (0)

// Per-device status word written by kernels whose bounded waits ran out.
// Allocated on first use for the current device; never freed.
int device_status_word(int** out);

// Maps a status word as the kernels write it (low byte: SILE_ERR_* code; bit 8 + n: wait site n
// was stuck) to the library's error: records the message and returns the code; 0 -> SILE_OK.
int decode_status_word(int word);

// The allocation-free matmul keeps its own status word inside the library image; this reads it
// into *value and clears it if it is non-zero (0 if that entry point was never used on the
// current device).
int noalloc_read_and_clear_status(int* value);

// A zero-initialisable work counter for one launch of a persistent kernel.  Counters come from a
// per-device pool of 1024 handed out round-robin; the launch resets its counter in stream order,
// so launches that overlap on different streams never share one unless more than 1024 launches
// are in flight on the device at once.  Allocated on first use; never freed.
int device_work_counter(int** out);

// Records the kernel a launch chose and its geometry for sile_cuda_last_kernel(), and prints it
// to stderr when SILE_PRINT_SOURCE, SILE_PRINT_LLVMIR or SILE_PRINT_TILEIR is set -- the
// reference dumps its generated source / IR under those names
// (crates/sile/src/kernel_launcher.rs:11-13,48-53); here the "source" is a hand-written kernel.
void note_kernel(const char* name, unsigned grid, unsigned block, size_t smem_bytes);

// cuTensorMapEncodeTiled through the runtime's driver entry-point lookup (no link
// dependency on libcuda).  Strides are in bytes and exclude the innermost one.
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle);

// ---- GEMM -----------------------------------------------------------------------
struct GemmProblem {
  const void* a = nullptr;   // [M,K] row-major, f32 or bf16/f16
  const void* b = nullptr;   // f32: [K,N] row-major; 16-bit: per b_layout
  void* c = nullptr;         // [M,N] row-major
  int64_t m = 0, n = 0, k = 0;
  int64_t ldc = 0;           // elements between rows of C; 0 = n
  int in_dtype = SILE_DTYPE_F32;
  int out_dtype = SILE_DTYPE_F32;
  int b_layout = SILE_LAYOUT_ROW_MAJOR;
  // Logical tile of the kernel definition and the number of launched tiles: they decide
  // which part of C is written (whole tiles only, K remainder dropped), never the CTA tiling.
  int64_t bm = 1, bn = 1, bk = 1;
  int64_t num_threadgroups = INT64_MAX;
  // D = C + A * B: the accumulator is seeded with what C holds (SILE_FLAG_ACCUMULATE).
  bool accumulate = false;
  // Fused all-gather: when num_peers > 0 every output element is stored into each peer_c[i]
  // (same layout and leading dimension as c) instead of c; peer_first rotates the order.
  void* peer_c[8] = {nullptr};
  int num_peers = 0;
  int peer_first = 0;
  void* workspace = nullptr;  // device scratch for the f32 split; see gemm_workspace_bytes
  size_t workspace_bytes = 0;
};
size_t gemm_workspace_bytes(const GemmProblem& p);
int gemm_launch(const GemmProblem& p, cudaStream_t stream);
// Text of the slice plan the sliced / all-gather GEMM kernel would take (host arithmetic only).
int gemm_slice_plan_text(int tiles, int clusters, int destinations, int exchange_bound, char* out, size_t cap);

// dst[r, j*cols + c] = src[j, r, c]: lays the rank-major result of an all-gather of column
// blocks out as one row-major matrix.
int unshard_columns_launch(void* dst, const void* src, int64_t parts, int64_t rows, int64_t cols, int elt_size,
                           cudaStream_t stream);

// Per-device caches (function attributes, occupancy) are arrays indexed by this: one process may
// drive several GPUs through sile_cuda_set_device.
constexpr int kMaxDevices = 64;
inline int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return dev;
}

// ---- attention forward ----------------------------------------------------------
struct AttnProblem {
  const void* q = nullptr;  // [BH, S, D] bf16
  const void* k = nullptr;  // [BH, S, D] bf16
  const void* v = nullptr;  // [BH, S, D] bf16
  void* o = nullptr;        // [BH, S, D] bf16
  int64_t bh = 0, s = 0, d = 0;
  float scale = 1.0f;
  int causal = 0;
  // Fused all-gather of O: when num_peers > 0 the bh heads computed here are heads
  // [bh_offset, bh_offset + bh) of peer_o[i] = rank i's [bh_total, S, D] buffer, and every rank's
  // buffer receives them (o is ignored).  Otherwise O goes to `o` only.
  int num_peers = 0;
  int peer_first = 0;  // destination served first (the local rank), then round-robin
  int64_t bh_total = 0, bh_offset = 0;
  void* peer_o[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
};
int attention_launch(const AttnProblem& p, cudaStream_t stream);
// CTA-pair kernel and persistent kernel; arguments already validated by attention_launch.
int attention_pair_launch(const AttnProblem& p, cudaStream_t stream);
int attention_persistent_launch(const AttnProblem& p, cudaStream_t stream);
int attention_split_launch(const AttnProblem& a, cudaStream_t stream);

// ---- standalone tile ops (HBM-bound) --------------------------------------------
int vec_add_launch(const float* a, const float* b, float* c, int64_t n, cudaStream_t stream);
int relu_launch(float* x, int64_t n, cudaStream_t stream);
int softmax_rows_launch(const float* x, int64_t ldx, float* y, int64_t ldy, int64_t rows, int64_t cols,
                        cudaStream_t stream);
int reduce_sum_launch(const float* a, int64_t n, float* out, cudaStream_t stream);
int matvec_launch(const float* x, const float* y, float* z, int64_t m, int64_t k, cudaStream_t stream);
// f32 <-> bf16 conversions around the bf16 attention kernel (n elements, n % 8 == 0), and the
// transposing one for K given as [BH][D][S] f32 -> [BH][S][D] bf16.
int cast_f32_to_bf16_launch(const float* src, void* dst, int64_t n, cudaStream_t stream);
int cast_bf16_to_f32_launch(const void* src, float* dst, int64_t n, cudaStream_t stream);
int transpose_cast_kt_launch(const float* kt, void* k, int64_t bh, int64_t s, int64_t d, cudaStream_t stream);
// Row softmax over column tiles: row r of tile column j (bn columns at x + r * ldx + j * bn) is
// normalised on its own, as the reference does for a [BM, BN] tile narrower than the row
// (crates/sile/examples/softmax.rs:3-16).  Only rows / tile columns whose logical tile id
// (r / bm) * tiles_n + j is below num_tiles are written.
int softmax_tiles_launch(const float* x, int64_t ldx, float* y, int64_t ldy, int64_t rows, int64_t tiles_n, int64_t bm,
                         int64_t bn, int64_t num_tiles, cudaStream_t stream);

}  // namespace sile
