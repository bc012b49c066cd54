// Standalone tile ops of the reference's examples as HBM-bound kernels:
// 128-bit vectorised, coalesced, grids sized in multiples of the SM count.
// Each replaces one generated scalar loop nest of the reference's lowering
// (crates/sile-tile-ir/src/passes/lowering/{tile_expr.rs,tile_compute/reduce.rs,
// tile_compute/fused_reduce.rs,block_scalar.rs}).
#include <cuda_bf16.h>

#include <algorithm>

#include "internal.h"

namespace sile {
namespace {

constexpr int kThreads = 256;

int sm_count() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

int grid_for(int64_t work_items, int per_sm) {
  const int sms = sm_count();
  const int64_t blocks = (work_items + kThreads - 1) / kThreads;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks, static_cast<int64_t>(sms) * per_sm)));
}

// c = a + b   (examples/vec_add.rs:3-10; tile_expr.rs pointwise store)
__global__ void vec_add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c, int64_t n, int vec) {
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    float4* c4 = reinterpret_cast<float4*>(c);
    for (int64_t i = tid; i < n4; i += nthreads) {
      const float4 x = __ldcs(a4 + i), y = __ldcs(b4 + i);
      __stcs(c4 + i, make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w));
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nthreads) c[i] = a[i] + b[i];
  } else {
    for (int64_t i = tid; i < n; i += nthreads) c[i] = a[i] + b[i];
  }
}

// x = max_tile(0, x) = (0 >= x) ? 0 : x   (lower.rs:619-641; examples/mlp.rs:51-55)
__device__ __forceinline__ float relu_sel(float v) { return (0.0f >= v) ? 0.0f : v; }
__global__ void relu_kernel(float* __restrict__ x, int64_t n, int vec) {
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    float4* x4 = reinterpret_cast<float4*>(x);
    for (int64_t i = tid; i < n4; i += nthreads) {
      float4 v = x4[i];
      v.x = relu_sel(v.x); v.y = relu_sel(v.y); v.z = relu_sel(v.z); v.w = relu_sel(v.w);
      x4[i] = v;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nthreads) x[i] = relu_sel(x[i]);
  } else {
    for (int64_t i = tid; i < n; i += nthreads) x[i] = relu_sel(x[i]);
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Row softmax (examples/softmax.rs:3-16): y = exp(x - max) / sum(exp(x - max)).
// One warp per row for short rows; the row is read once from HBM when it fits the
// per-lane register cache (cols <= 32 * kCache), otherwise it is re-read from L2.
constexpr int kCache = 32;
__global__ void softmax_rows_kernel(const float* __restrict__ x, int64_t ldx, float* __restrict__ y, int64_t ldy, int64_t rows,
                                    int cols) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t warp_global = blockIdx.x * static_cast<int64_t>(warps_per_block) + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps_per_block;
  for (int64_t row = warp_global; row < rows; row += nwarps) {
    const float* xr = x + row * ldx;
    float* yr = y + row * ldy;
    float cache[kCache];
    const bool cached = cols <= 32 * kCache;
    float mx = -INFINITY;
    if (cached) {
#pragma unroll
      for (int i = 0; i < kCache; ++i) {
        const int c = lane + 32 * i;
        cache[i] = c < cols ? xr[c] : -INFINITY;
        mx = fmaxf(mx, cache[i]);
      }
    } else {
      for (int c = lane; c < cols; c += 32) mx = fmaxf(mx, xr[c]);
    }
    mx = warp_max(mx);
    float sum = 0.0f;
    if (cached) {
#pragma unroll
      for (int i = 0; i < kCache; ++i) {
        const int c = lane + 32 * i;
        cache[i] = c < cols ? expf(cache[i] - mx) : 0.0f;
        sum += cache[i];
      }
    } else {
      for (int c = lane; c < cols; c += 32) sum += expf(xr[c] - mx);
    }
    sum = warp_sum(sum);
    if (cached) {
#pragma unroll
      for (int i = 0; i < kCache; ++i) {
        const int c = lane + 32 * i;
        if (c < cols) yr[c] = cache[i] / sum;
      }
    } else {
      for (int c = lane; c < cols; c += 32) yr[c] = expf(xr[c] - mx) / sum;
    }
  }
}

// Tile-local softmax: the reference normalises each [BM, BN] tile on its own
// (examples/softmax.rs:3-16), so with BN smaller than the row every BN-wide segment of a row is a
// softmax of its own.  One warp per (row, tile column) segment; a segment is written only if its
// logical tile (row / bm) * tiles_n + tile column was launched (cpu/codegen.rs:517-533).
__global__ void softmax_tiles_kernel(const float* __restrict__ x, int64_t ldx, float* __restrict__ y, int64_t ldy, int64_t rows,
                                     int tiles_n, int bm, int bn, int64_t num_tiles) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t warp_global = blockIdx.x * static_cast<int64_t>(warps_per_block) + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps_per_block;
  const int64_t segments = rows * tiles_n;
  for (int64_t seg = warp_global; seg < segments; seg += nwarps) {
    const int64_t r = seg / tiles_n;
    const int jt = static_cast<int>(seg - r * tiles_n);
    if ((r / bm) * tiles_n + jt >= num_tiles) continue;
    const float* xr = x + r * ldx + static_cast<int64_t>(jt) * bn;
    float* yr = y + r * ldy + static_cast<int64_t>(jt) * bn;
    float mx = -INFINITY;
    for (int c = lane; c < bn; c += 32) mx = fmaxf(mx, xr[c]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int c = lane; c < bn; c += 32) sum += expf(xr[c] - mx);
    sum = warp_sum(sum);
    for (int c = lane; c < bn; c += 32) yr[c] = expf(xr[c] - mx) / sum;
  }
}

// Rows of up to 128 * kChunks columns with 16-byte aligned rows: each lane holds kChunks float4
// (the row is read once, 512 bytes per warp load), all loads of a row are issued before the first
// use, exp is ex2.approx on (x - max) * log2(e) and the division becomes one reciprocal per row.
template <int kChunks>
__global__ void softmax_rows_vec4_kernel(const float* __restrict__ x, int64_t ldx, float* __restrict__ y, int64_t ldy, int64_t rows,
                                         int cols4) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t warp_global = blockIdx.x * static_cast<int64_t>(warps_per_block) + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps_per_block;
  constexpr float kLog2e = 1.4426950408889634f;
  for (int64_t row = warp_global; row < rows; row += nwarps) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * ldx);
    float4* yr = reinterpret_cast<float4*>(y + row * ldy);
    float4 v[kChunks];
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
      const int c = lane + 32 * i;
      v[i] = c < cols4 ? __ldcs(xr + c) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kChunks; ++i) mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    mx = warp_max(mx);
    const float off = mx * kLog2e;
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
      v[i].x = exp2f(fmaf(v[i].x, kLog2e, -off));
      v[i].y = exp2f(fmaf(v[i].y, kLog2e, -off));
      v[i].z = exp2f(fmaf(v[i].z, kLog2e, -off));
      v[i].w = exp2f(fmaf(v[i].w, kLog2e, -off));
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
      const int c = lane + 32 * i;
      if (c < cols4) __stcs(yr + c, make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv));
    }
  }
}

// out[0] += sum(a[0..n))   (examples/parallel_reduce.rs:3-9: per-tile reduce_sum then
// atomic_add; block_scalar.rs:98-157).  One red.global.add.f32 per block; the order of
// the atomics is nondeterministic here as it is under OpenMP in the reference.
__global__ void reduce_sum_kernel(const float* __restrict__ a, int64_t n, float* __restrict__ out, int vec) {
  __shared__ float partial[32];
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  float acc = 0.0f;
  if (vec) {
    const int64_t n4 = n >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    float acc2 = 0.0f;
    int64_t i = tid;
    for (; i + nthreads < n4; i += 2 * nthreads) {
      const float4 v = __ldcs(a4 + i);
      const float4 w = __ldcs(a4 + i + nthreads);
      acc += (v.x + v.y) + (v.z + v.w);
      acc2 += (w.x + w.y) + (w.z + w.w);
    }
    for (; i < n4; i += nthreads) {
      const float4 v = __ldcs(a4 + i);
      acc += (v.x + v.y) + (v.z + v.w);
    }
    acc += acc2;
    for (int64_t j = (n4 << 2) + tid; j < n; j += nthreads) acc += a[j];
  } else {
    for (int64_t i = tid; i < n; i += nthreads) acc += a[i];
  }
  acc = warp_sum(acc);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) partial[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    float v = lane < (blockDim.x >> 5) ? partial[lane] : 0.0f;
    v = warp_sum(v);
    if (lane == 0) atomicAdd(out, v);
  }
}

// z[r] = sum_k x[r,k] * y[k]   (examples/mlp.rs:28-46).  One warp per row, float4 loads.
__global__ void matvec_kernel(const float* __restrict__ x, const float* __restrict__ y, float* __restrict__ z, int64_t m, int64_t k,
                              int vec) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t warp_global = blockIdx.x * static_cast<int64_t>(warps_per_block) + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps_per_block;
  for (int64_t row = warp_global; row < m; row += nwarps) {
    const float* xr = x + row * k;
    float acc = 0.0f;
    if (vec) {
      const int64_t k4 = k >> 2;
      const float4* x4 = reinterpret_cast<const float4*>(xr);
      const float4* y4 = reinterpret_cast<const float4*>(y);
      for (int64_t i = lane; i < k4; i += 32) {
        const float4 a = __ldcs(x4 + i);
        const float4 b = __ldg(y4 + i);
        acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
      }
    } else {
      for (int64_t i = lane; i < k; i += 32) acc += xr[i] * y[i];
    }
    acc = warp_sum(acc);
    if (lane == 0) z[row] = acc;
  }
}

// K <= 128 * kChunks, 16-byte aligned: the lane's share of y stays in registers for every row the
// warp handles, and two rows are in flight per step (all their loads issued before the first FMA).
template <int kChunks>
__global__ void matvec_vec4_kernel(const float* __restrict__ x, const float* __restrict__ y, float* __restrict__ z, int64_t m, int k4) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t warp_global = blockIdx.x * static_cast<int64_t>(warps_per_block) + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps_per_block;
  const float4* y4 = reinterpret_cast<const float4*>(y);
  float4 yv[kChunks];
#pragma unroll
  for (int i = 0; i < kChunks; ++i) {
    const int c = lane + 32 * i;
    yv[i] = c < k4 ? __ldg(y4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int64_t row = 2 * warp_global; row < m; row += 2 * nwarps) {
    const float4* x0 = reinterpret_cast<const float4*>(x) + row * k4;
    const bool two = row + 1 < m;
    const float4* x1 = x0 + (two ? k4 : 0);
    float4 a[kChunks], b[kChunks];
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
      const int c = lane + 32 * i;
      a[i] = c < k4 ? __ldcs(x0 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      b[i] = c < k4 ? __ldcs(x1 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
      acc0 += a[i].x * yv[i].x + a[i].y * yv[i].y + a[i].z * yv[i].z + a[i].w * yv[i].w;
      acc1 += b[i].x * yv[i].x + b[i].y * yv[i].y + b[i].z * yv[i].z + b[i].w * yv[i].w;
    }
    acc0 = warp_sum(acc0);
    acc1 = warp_sum(acc1);
    if (lane == 0) {
      z[row] = acc0;
      if (two) z[row + 1] = acc1;
    }
  }
}

// dst[r][j*cols + c] = src[j][r][c], 16 bytes per thread per step.
__global__ void unshard_columns_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int parts, int64_t rows, int cols16) {
  const int64_t per_part = rows * cols16;
  const int64_t total = per_part * parts;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t j = i / per_part;
    const int64_t rem = i - j * per_part;
    const int64_t r = rem / cols16;
    const int64_t c = rem - r * cols16;
    __stcs(dst + (r * parts + j) * cols16 + c, __ldcs(src + i));
  }
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// ---- dtype / layout conversions around the bf16 attention kernel ---------------------------------
// The reference's tensors are f32 and its DSL has no transpose, so an attention kernel composed
// from its tile ops receives Q, V as [B*H*S, D] and K already transposed as [B*H*D, S]
// (crates/sile-tile-ir/src/passes/lowering/tile_memory.rs:164-228: rank-2 row-major tiles only).
// These kernels bring such buffers into the [B*H, S, D] bf16 layout the tensor-core kernel reads,
// and its bf16 output back to f32.  HBM-bound: 16-byte accesses, 6 bytes per element.
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n8) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i);
    const float4 b = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i + 1);
    uint4 o;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(a.x, a.y); o.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(a.z, a.w); o.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(b.x, b.y); o.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(b.z, b.w); o.w = *reinterpret_cast<uint32_t*>(&t);
    reinterpret_cast<uint4*>(dst)[i] = o;
  }
}

__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, int64_t n8) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(src)[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      f[2 * h] = __uint_as_float(w[h] << 16);
      f[2 * h + 1] = __uint_as_float(w[h] & 0xffff0000u);
    }
    __stcs(reinterpret_cast<float4*>(dst) + 2 * i, make_float4(f[0], f[1], f[2], f[3]));
    __stcs(reinterpret_cast<float4*>(dst) + 2 * i + 1, make_float4(f[4], f[5], f[6], f[7]));
  }
}

// kt [BH][D][S] f32 -> k [BH][S][D] bf16.  Block = 32 x 8 threads, tile = 64 (d) x 32 (s): reads run
// along s, writes along d (two elements per thread, 128 bytes per warp).
__global__ void transpose_cast_kt_kernel(const float* __restrict__ kt, __nv_bfloat16* __restrict__ k, int s, int d) {
  __shared__ float tile[64][33];
  const int s0 = blockIdx.x * 32, d0 = blockIdx.y * 64;
  const int64_t head = blockIdx.z;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const float* src = kt + head * static_cast<int64_t>(d) * s;
  __nv_bfloat16* dst = k + head * static_cast<int64_t>(s) * d;
#pragma unroll
  for (int dd = ty; dd < 64; dd += 8) {
    const int di = d0 + dd, si = s0 + tx;
    tile[dd][tx] = (di < d && si < s) ? __ldcs(src + static_cast<int64_t>(di) * s + si) : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for (int ss = ty; ss < 32; ss += 8) {
    const int si = s0 + ss, di = d0 + 2 * tx;
    if (si < s && di + 1 < d) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(tile[2 * tx][ss], tile[2 * tx + 1][ss]);
      *reinterpret_cast<__nv_bfloat162*>(dst + static_cast<int64_t>(si) * d + di) = v;
    }
  }
}

}  // namespace

int cast_f32_to_bf16_launch(const float* src, void* dst, int64_t n, cudaStream_t stream) {
  if (n <= 0) return SILE_OK;
  if (n % 8 != 0 || !aligned16(src) || !aligned16(dst)) return fail(SILE_ERR_UNSUPPORTED, "cast: element count must be a multiple of 8 and buffers 16-byte aligned");
  cast_f32_to_bf16_kernel<<<grid_for(n / 8, 8), kThreads, 0, stream>>>(src, static_cast<__nv_bfloat16*>(dst), n / 8);
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

int cast_bf16_to_f32_launch(const void* src, float* dst, int64_t n, cudaStream_t stream) {
  if (n <= 0) return SILE_OK;
  if (n % 8 != 0 || !aligned16(src) || !aligned16(dst)) return fail(SILE_ERR_UNSUPPORTED, "cast: element count must be a multiple of 8 and buffers 16-byte aligned");
  cast_bf16_to_f32_kernel<<<grid_for(n / 8, 8), kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), dst, n / 8);
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

int transpose_cast_kt_launch(const float* kt, void* k, int64_t bh, int64_t s, int64_t d, cudaStream_t stream) {
  if (bh <= 0 || s <= 0 || d <= 0) return SILE_OK;
  if (d % 2 != 0 || bh > 65535) return fail(SILE_ERR_UNSUPPORTED, "attention: head_dim must be even and batch*heads at most 65535 for f32 inputs");
  dim3 grid(static_cast<unsigned>((s + 31) / 32), static_cast<unsigned>((d + 63) / 64), static_cast<unsigned>(bh));
  transpose_cast_kt_kernel<<<grid, dim3(32, 8), 0, stream>>>(kt, static_cast<__nv_bfloat16*>(k), static_cast<int>(s), static_cast<int>(d));
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

int unshard_columns_launch(void* dst, const void* src, int64_t parts, int64_t rows, int64_t cols, int elt_size,
                           cudaStream_t stream) {
  if (parts <= 0 || rows <= 0 || cols <= 0) return SILE_OK;
  if (!dst || !src) return fail(SILE_ERR_INVALID, "unshard: null buffer");
  if ((cols * elt_size) % 16 != 0 || !aligned16(dst) || !aligned16(src))
    return fail(SILE_ERR_UNSUPPORTED, "unshard: column blocks must be multiples of 16 bytes and 16-byte aligned");
  const int64_t cols16 = cols * elt_size / 16;
  unshard_columns_kernel<<<grid_for(parts * rows * cols16, 8), kThreads, 0, stream>>>(
      static_cast<uint4*>(dst), static_cast<const uint4*>(src), static_cast<int>(parts), rows, static_cast<int>(cols16));
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

int vec_add_launch(const float* a, const float* b, float* c, int64_t n, cudaStream_t stream) {
  if (n <= 0) return SILE_OK;
  const int vec = aligned16(a) && aligned16(b) && aligned16(c);
  vec_add_kernel<<<grid_for((n + 3) / 4, 8), kThreads, 0, stream>>>(a, b, c, n, vec);
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

int relu_launch(float* x, int64_t n, cudaStream_t stream) {
  if (n <= 0) return SILE_OK;
  relu_kernel<<<grid_for((n + 3) / 4, 8), kThreads, 0, stream>>>(x, n, aligned16(x));
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

int softmax_rows_launch(const float* x, int64_t ldx, float* y, int64_t ldy, int64_t rows, int64_t cols, cudaStream_t stream) {
  if (rows <= 0) return SILE_OK;
  if (cols > (1ll << 30)) return fail(SILE_ERR_INVALID, "softmax: row too long");
  const bool vec = cols % 4 == 0 && cols <= 1024 && ldx % 4 == 0 && ldy % 4 == 0 && aligned16(x) && aligned16(y);
  if (vec) {
    const int cols4 = static_cast<int>(cols / 4);
    const int grid = grid_for(rows * 32, 8);
    if (cols4 <= 32) softmax_rows_vec4_kernel<1><<<grid, kThreads, 0, stream>>>(x, ldx, y, ldy, rows, cols4);
    else if (cols4 <= 64) softmax_rows_vec4_kernel<2><<<grid, kThreads, 0, stream>>>(x, ldx, y, ldy, rows, cols4);
    else if (cols4 <= 128) softmax_rows_vec4_kernel<4><<<grid, kThreads, 0, stream>>>(x, ldx, y, ldy, rows, cols4);
    else softmax_rows_vec4_kernel<8><<<grid, kThreads, 0, stream>>>(x, ldx, y, ldy, rows, cols4);
  } else {
    softmax_rows_kernel<<<grid_for(rows * 32, 8), kThreads, 0, stream>>>(x, ldx, y, ldy, rows, static_cast<int>(cols));
  }
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

int softmax_tiles_launch(const float* x, int64_t ldx, float* y, int64_t ldy, int64_t rows, int64_t tiles_n, int64_t bm, int64_t bn,
                         int64_t num_tiles, cudaStream_t stream) {
  if (rows <= 0 || tiles_n <= 0 || num_tiles <= 0) return SILE_OK;
  if (bn > (1ll << 30) || tiles_n > (1ll << 30) || bm > (1ll << 30)) return fail(SILE_ERR_INVALID, "softmax: tile too large");
  softmax_tiles_kernel<<<grid_for(rows * tiles_n * 32, 8), kThreads, 0, stream>>>(x, ldx, y, ldy, rows, static_cast<int>(tiles_n),
                                                                                 static_cast<int>(bm), static_cast<int>(bn), num_tiles);
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

int reduce_sum_launch(const float* a, int64_t n, float* out, cudaStream_t stream) {
  if (n <= 0) return SILE_OK;
  reduce_sum_kernel<<<grid_for((n + 3) / 4, 4), kThreads, 0, stream>>>(a, n, out, aligned16(a));
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

int matvec_launch(const float* x, const float* y, float* z, int64_t m, int64_t k, cudaStream_t stream) {
  if (m <= 0) return SILE_OK;
  const int vec = aligned16(x) && aligned16(y) && (k % 4 == 0);
  if (vec && k <= 1024) {
    const int k4 = static_cast<int>(k / 4);
    const int grid = grid_for((m + 1) / 2 * 32, 8);
    if (k4 <= 32) matvec_vec4_kernel<1><<<grid, kThreads, 0, stream>>>(x, y, z, m, k4);
    else if (k4 <= 64) matvec_vec4_kernel<2><<<grid, kThreads, 0, stream>>>(x, y, z, m, k4);
    else if (k4 <= 128) matvec_vec4_kernel<4><<<grid, kThreads, 0, stream>>>(x, y, z, m, k4);
    else matvec_vec4_kernel<8><<<grid, kThreads, 0, stream>>>(x, y, z, m, k4);
  } else {
    matvec_kernel<<<grid_for(m * 32, 8), kThreads, 0, stream>>>(x, y, z, m, k, vec);
  }
  SILE_CUDA_TRY(cudaGetLastError());
  return SILE_OK;
}

}  // namespace sile
