// Tiled dense contraction C[M,N] = A[M,K] * B[K,N] for sm_100a.
//
// The hand-written counterpart of the reference's generated canonical matmul
// (crates/sile-tile-ir/src/passes/lowering/canonical_matmul.rs:24-444) and of its
// OpenMP tile loop (crates/sile-backend/src/cpu/codegen.rs:517-551).
//
// Four persistent, warp-specialised kernels share one structure -- warp 0 TMA producer (global ->
// 128B-swizzled shared-memory ring), warp 1 tcgen05.mma kind::f16 issuer with f32 accumulators in
// TMEM, the remaining warps epilogue (tcgen05.ld -> convert -> global):
//   gemm_tn_kernel            one CTA, 128 x 256 x 64 tiles, two accumulators
//   gemm_tn_pair_kernel       CTA pair (cta_group::2), 256 x 256 x 64, two accumulators
//   gemm_tn_pair_wide_kernel  CTA pair, 256 x 512 x 64, one accumulator, TMA-store epilogue
//   gemm_tn_pair_sliced_kernel  CTA pair, 256 x 256 x 64 tiles that can be cut into column slices,
//                             two accumulators, TMA stores to one or to every rank's C (all-gather)
// gemm_launch picks one by problem shape; see the comments at each kernel.
//
// f32 inputs are not fed to the tensor cores as tf32.  Each f32 value x is split
// into bf16 hi = rn(x) and lo = rn(x - hi); the product is formed as
// hi*hi + hi*lo + lo*hi with f32 accumulation, i.e. ONE bf16 GEMM over a
// three-segment K axis.  The dropped lo*lo term and the split residue are
// ~2^-17 relative per product, far inside the 1e-3 bound on max-abs error
// relative to output scale.  The split (and B's transpose to K-major) is a
// separate HBM-bound pre-pass into caller-provided scratch.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>
#include <vector>

#include "internal.h"
#include "ptx.cuh"

namespace sile {
namespace {

using namespace ptx;

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;  // 64 x 16-bit = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK * 2;
constexpr int kBBytes = kBN * kBK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;
constexpr int kNumThreads = 192;
constexpr int kGroupM = 16;  // m-blocks per raster group: one wave shares A rows / B columns in L2
constexpr int kSmemBytes = kStages * kStageBytes + 256 /*barriers*/ + 1024 /*alignment slack*/;

struct GemmParams {
  int m_valid;        // rows of C that may be written (whole logical tiles only)
  int n_valid;        // columns of C that may be written
  int64_t ldc;
  int m_blocks, n_blocks;
  int k_blocks_per_seg;  // 64-wide k blocks per segment
  int num_segs;          // 1 (16-bit inputs) or 3 (split f32)
  int a_seg_row[3];      // row offset of each segment's A operand in the A tensor map
  int b_seg_row[3];      // row offset of each segment's B operand in the B tensor map
  // launch mask of the logical grid: element (r,c) belongs to logical tile
  // (r / lbm) * ltiles_n + c / lbn and is written only if that id < ntg.
  int lbm, lbn, ltiles_n;
  long long ntg;
  int masked;  // 1 if the logical launch mask can exclude anything
  int group_m;  // 128-row blocks per raster group
  // 1: the accumulator is seeded with the output tile, D = C + A * B -- the general mma of the
  // reference (`sum0 = acc[r][c]`, tile_compute/mma.rs:25-260) with acc loaded from the output;
  // the epilogue adds the value C held to the tensor-core sum before storing.
  int accumulate;
};

// Destinations of the wide kernel's epilogue.  Normally one (the caller's C); for the fused
// GEMM + all-gather every rank's buffer is listed (this GPU's own and its peers', reached over
// NVLink through peer-mapped pointers) and every output element is stored into each of them,
// starting with `first` so that ranks do not all hit the same peer at once.
struct PeerOut {
  void* ptr[8];  // same layout and leading dimension as C, already offset to the column block
  int count;     // >= 1
  int first;
};
// One tensor map per destination for the epilogue's TMA stores: 2-D {columns, rows} over the
// destination starting at its column block, box = 128 bytes x 32 rows, 128-byte swizzle.
struct OutMaps {
  CUtensorMap map[8];
};

__device__ __forceinline__ void tile_coords(int t, const GemmParams& p, int& m_blk, int& n_blk) {
  const int group_m = p.group_m;
  const int group_size = group_m * p.n_blocks;
  const int group = t / group_size;
  const int first_m = group * group_m;
  const int gm = min(p.m_blocks - first_m, group_m);
  const int r = t - group * group_size;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* c, const GemmParams& p, int row, int col0, const uint32_t (&r)[32], bool fast) {
  // Thread owns 32 consecutive columns [col0, col0+32) of `row`.
  if (fast) {
    if constexpr (sizeof(OutT) == 4) {
      float4* dst = reinterpret_cast<float4*>(c + static_cast<int64_t>(row) * p.ldc + col0);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                               __uint_as_float(r[4 * i + 3]));
        if (p.accumulate) {
          const float4 old = dst[i];
          v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
        }
        dst[i] = v;
      }
    } else {
      uint4* dst = reinterpret_cast<uint4*>(c + static_cast<int64_t>(row) * p.ldc + col0);
      float f[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
      if (p.accumulate) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 old = dst[i];
          const uint32_t w[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
              f[8 * i + 2 * h] += __uint_as_float(w[h] << 16);
              f[8 * i + 2 * h + 1] += __uint_as_float(w[h] & 0xffff0000u);
            } else {
              const __half2 hv = *reinterpret_cast<const __half2*>(&w[h]);
              f[8 * i + 2 * h] += __low2float(hv);
              f[8 * i + 2 * h + 1] += __high2float(hv);
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 v;
        if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
          v.x = pack_bf16x2(f[8 * i], f[8 * i + 1]);
          v.y = pack_bf16x2(f[8 * i + 2], f[8 * i + 3]);
          v.z = pack_bf16x2(f[8 * i + 4], f[8 * i + 5]);
          v.w = pack_bf16x2(f[8 * i + 6], f[8 * i + 7]);
        } else {
          __half2 h0 = __floats2half2_rn(f[8 * i], f[8 * i + 1]);
          __half2 h1 = __floats2half2_rn(f[8 * i + 2], f[8 * i + 3]);
          __half2 h2 = __floats2half2_rn(f[8 * i + 4], f[8 * i + 5]);
          __half2 h3 = __floats2half2_rn(f[8 * i + 6], f[8 * i + 7]);
          v.x = *reinterpret_cast<uint32_t*>(&h0);
          v.y = *reinterpret_cast<uint32_t*>(&h1);
          v.z = *reinterpret_cast<uint32_t*>(&h2);
          v.w = *reinterpret_cast<uint32_t*>(&h3);
        }
        dst[i] = v;
      }
    }
    return;
  }
  if (row >= p.m_valid) return;
  const long long tile_row = static_cast<long long>(row / p.lbm) * p.ltiles_n;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int col = col0 + i;
    if (col < p.n_valid && (!p.masked || tile_row + col / p.lbn < p.ntg)) {
      float v = __uint_as_float(r[i]);
      OutT* dst = c + static_cast<int64_t>(row) * p.ldc + col;
      if (p.accumulate) {
        if constexpr (sizeof(OutT) == 4) v += *dst;
        else if constexpr (std::is_same<OutT, __nv_bfloat16>::value) v += __bfloat162float(*dst);
        else v += __half2float(*dst);
      }
      if constexpr (sizeof(OutT) == 4) {
        *dst = v;
      } else if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
        *dst = __float2bfloat16_rn(v);
      } else {
        *dst = __float2half_rn(v);
      }
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, OutT* __restrict__ c,
               const GemmParams p, const uint32_t idesc, const int vec_ok, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 4);  // one arrival per epilogue warp
    }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, kTmemCols);
    tmem_relinquish<1>();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  const int num_tiles = p.m_blocks * p.n_blocks;
  const int num_kb = p.k_blocks_per_seg * p.num_segs;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(t, p, m_blk, n_blk);
        int seg = 0, kb_in_seg = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, status, SILE_ERR_TIMEOUT)) { ok = false; break; }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          tma_load_2d(sa, &tma_a, &full_bar[stage], kb_in_seg * kBK, p.a_seg_row[seg] + m_blk * kBM);
          tma_load_2d(sb, &tma_b, &full_bar[stage], kb_in_seg * kBK, p.b_seg_row[seg] + n_blk * kBN);
          if (++kb_in_seg == p.k_blocks_per_seg) { kb_in_seg = 0; ++seg; }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp runs the loop; the tcgen05 instructions are predicated on one elected lane
    // (see umma_ss_f16_if), which keeps descriptor arithmetic in the uniform datapath.
    {
      const uint32_t el = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&tmem_empty_bar[buf], acc_phase ^ 1u, status, SILE_ERR_TIMEOUT))) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, status, SILE_ERR_TIMEOUT))) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sa + kABytes, 16, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // +32 bytes per 16-element k step inside the 128-byte swizzle row (address field is >>4)
            umma_ss_f16_if<1>(el, tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_if<1>(el, smem_u32(&empty_bar[stage]));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_if<1>(el, smem_u32(&tmem_full_bar[buf]));
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are this warp's
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      int m_blk, n_blk;
      tile_coords(t, p, m_blk, n_blk);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full_bar[buf], acc_phase, status, SILE_ERR_TIMEOUT)) { ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = m_blk * kBM + quarter * 32 + lane;
      const int col_base = n_blk * kBN;
      const bool tile_fast = vec_ok && !p.masked && (m_blk * kBM + kBM <= p.m_valid) && (col_base + kBN <= p.n_valid);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBN;
#pragma unroll 1
      for (int ch = 0; ch < kBN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + ch * 32, r);
        tcgen05_wait_ld();
        if (tile_fast || col_base + ch * 32 < p.n_valid) store_chunk<OutT>(c, p, row, col_base + ch * 32, r, tile_fast);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    if (*reinterpret_cast<volatile int*>(status) != 0) {
      // A wait ran out somewhere: give copies and MMAs still in flight time to land
      // before the accumulators are released.
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {
      }
    }
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

// ---- CTA-pair variant ---------------------------------------------------------------
// Two CTAs of a cluster share one 256 x 256 x 64 tile: CTA r stages rows [128r, 128r+128) of A
// and rows [128r, 128r+128) of the B tile (16 KiB + 16 KiB per stage, 6 stages), the leader
// (cluster rank 0) issues tcgen05.mma.cta_group::2 with M = 256, N = 256 and each CTA's TMEM
// receives its 128 accumulator rows.  Every TMA load completes on the LEADER's full barrier;
// the leader's commits release the stage, and publish the accumulator, in both CTAs; both
// CTAs' epilogue warps report to the leader's tmem_empty barrier.  Every load is a plain per-CTA TMA load.
constexpr int kPairStages = 6;
constexpr int kPairABytes = 128 * kBK * 2;
constexpr int kPairBBytes = 128 * kBK * 2;
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 256 + 1024;
constexpr int kPairBM = 256;

__device__ __forceinline__ void pair_tile_coords(int t, const GemmParams& p, int m_blocks, int& m_blk, int& n_blk) {
  const int kGroup = max(p.group_m / 2, 1);
  const int group_size = kGroup * p.n_blocks;
  const int group = t / group_size;
  const int first_m = group * kGroup;
  const int gm = min(m_blocks - first_m, kGroup);
  const int r = t - group * group_size;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

template <typename OutT>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tn_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, OutT* __restrict__ c,
                    const GemmParams p, const uint32_t idesc, const int vec_ok, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  uint64_t* empty_bar = full_bar + kPairStages;
  uint64_t* tmem_full_bar = empty_bar + kPairStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 8);  // 4 epilogue warps in each of the two CTAs
    }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, kTmemCols);
    tmem_relinquish<2>();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is signalled across CTAs
  tcgen05_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  const int m_blocks = (p.m_valid + kPairBM - 1) / kPairBM;
  const int num_tiles = m_blocks * p.n_blocks;
  const int num_kb = p.k_blocks_per_seg * p.num_segs;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int m_blk, n_blk;
        pair_tile_coords(t, p, m_blocks, m_blk, n_blk);
        const int a_row = m_blk * kPairBM + static_cast<int>(rank) * 128;
        const int b_row = n_blk * kBN + static_cast<int>(rank) * 128;
        int seg = 0, kb_in_seg = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait<true>(&empty_bar[stage], phase ^ 1u, status, SILE_ERR_TIMEOUT, 1 + 4 * rank)) { ok = false; break; }
          uint8_t* sa = smem + stage * kPairStageBytes;
          uint8_t* sb = sa + kPairABytes;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kPairStageBytes);
          tma_load_2d_pair(sa, &tma_a, &full_bar[stage], 0, kb_in_seg * kBK, p.a_seg_row[seg] + a_row);
          tma_load_2d_pair(sb, &tma_b, &full_bar[stage], 0, kb_in_seg * kBK, p.b_seg_row[seg] + b_row);
          if (++kb_in_seg == p.k_blocks_per_seg) { kb_in_seg = 0; ++seg; }
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    // Whole warp, predicated tcgen05 instructions: see umma_ss_f16_if.
    if (leader) {
      const uint32_t el = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait<true>(&tmem_empty_bar[buf], acc_phase ^ 1u, status, SILE_ERR_TIMEOUT, 2))) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait<true>(&full_bar[stage], phase, status, SILE_ERR_TIMEOUT, 3))) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kPairStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sa + kPairABytes, 16, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) umma_ss_f16_if<2>(el, tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_if<2>(el, pair_addr(&empty_bar[stage], 0));
          umma_commit_if<2>(el, pair_addr(&empty_bar[stage], 1));
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          umma_commit_if<2>(el, pair_addr(&tmem_full_bar[buf], 0));
          umma_commit_if<2>(el, pair_addr(&tmem_full_bar[buf], 1));
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (both CTAs) ----------------
    const int quarter = warp & 3;
    int it = 0;
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++it) {
      int m_blk, n_blk;
      pair_tile_coords(t, p, m_blocks, m_blk, n_blk);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait<true>(&tmem_full_bar[buf], acc_phase, status, SILE_ERR_TIMEOUT, 4 + 4 * rank)) { ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row0 = m_blk * kPairBM + static_cast<int>(rank) * 128;
      const int row = row0 + quarter * 32 + lane;
      const int col_base = n_blk * kBN;
      const bool tile_fast = vec_ok && !p.masked && (row0 + 128 <= p.m_valid) && (col_base + kBN <= p.n_valid);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBN;
#pragma unroll 1
      for (int ch = 0; ch < kBN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + ch * 32, r);
        tcgen05_wait_ld();
        if (tile_fast || col_base + ch * 32 < p.n_valid) store_chunk<OutT>(c, p, row, col_base + ch * 32, r, tile_fast);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(&tmem_empty_bar[buf], 0);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still touch its shared memory or TMEM
  if (warp == 1) {
    tcgen05_fence_after();
    if (*reinterpret_cast<volatile int*>(status) != 0) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {
      }
    }
    tmem_dealloc<2>(tmem_base, kTmemCols);
  }
}

// ---- CTA-pair variant with sliced tiles and a TMA-store epilogue for one or many destinations ----
// The 256 x 256 pair kernel above with a store epilogue built for the fused all-gather: each
// epilogue warp converts its 32 rows of a tile box by box (128 bytes x 32 rows, 128-byte swizzle)
// through two staging boxes of its own, and lane 0 issues one TMA store per box and DESTINATION
// -- this GPU's C and every peer's, over NVLink -- starting with a different destination for
// every item.  The tile has two accumulators, so the stores of tile i are issued and drain while
// tile i+1 is being computed; a box is only waited for (for shared memory to have been read) when
// its staging slot comes round again, two boxes later.  The ring keeps the six 32 KiB stages of
// the plain pair kernel; with four (a first version, with a whole-tile staging buffer instead)
// the main loop ran out of data in flight and the kernel was no faster than the wide one.
// With a single destination it is also the fastest kernel for shapes whose 256 x 512 tiles fill
// the CTA pairs' waves badly (gemm_launch compares the two).
//
// Work items are tiles or column slices of tiles, in consecutive groups each cut into 2^s slices
// of 256 >> s columns (s = 0, 1 or 2): a slice is an MMA of that N fed by (128 >> s) rows of B per
// CTA and stored as (4 >> s) boxes per warp (16-bit outputs; twice as many 32-column boxes for
// f32).  Item i goes to CTA pair i mod (pairs).  Slicing the tiles of
// the last, partly filled wave halves the time that wave takes (256 tiles on 74 CTA pairs are 3.5
// waves instead of 4); with several destinations a few sliced tiles at the head put the CTA
// pairs out of step with one another, so that their store bursts do not all hit NVLink at once.
constexpr int kAgStages = 6;
constexpr int kAgStagingBytes = 4 * 2 * 4096;  // 4 epilogue warps x 2 boxes of 32 rows x 128 bytes
constexpr int kAgSmemBytes = kAgStages * kPairStageBytes + kAgStagingBytes + 256 + 1024;

// B through three tensor maps whose boxes are a CTA's share of a whole tile, a half and a quarter
// (128, 64, 32 rows): one load per stage whatever the slice.  (Loading a whole tile's share as four
// 32-row boxes cost a fifth of the kernel's throughput.)
struct AgBMaps {
  CUtensorMap map[3];
};

constexpr int kAgMaxGroups = 6;
struct AgPlan {
  int groups;               // consecutive groups of tiles, each cut its own way
  int n[kAgMaxGroups];      // tiles per group (the last group takes what is left)
  int s[kAgMaxGroups];      // log2 of the slices per tile
  int items;                // sum of n[g] << s[g]
  uint32_t idesc[3];        // instruction descriptors for N = 256, 128, 64
};

__device__ __forceinline__ void ag_item(int i, const AgPlan& plan, int& tile, int& part, int& s) {
  int first = 0, g = 0;  // first tile of the group item i falls in
  while (g + 1 < plan.groups && i >= (plan.n[g] << plan.s[g])) {
    i -= plan.n[g] << plan.s[g];
    first += plan.n[g];
    ++g;
  }
  s = plan.s[g];
  tile = first + (i >> s);
  part = i - ((i >> s) << s);
}

template <typename OutT>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tn_pair_sliced_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ AgBMaps tma_b, const GemmParams p,
                       const AgPlan plan, const int vec_ok, int* __restrict__ status, const PeerOut peers,
                       const __grid_constant__ OutMaps out_maps) {
  constexpr int kBoxCols = 128 / static_cast<int>(sizeof(OutT));  // columns in a 128-byte store box
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + kAgStages * kPairStageBytes;  // 1024-byte aligned: matches the store maps' swizzle
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + kAgStagingBytes);
  uint64_t* empty_bar = full_bar + kAgStages;
  uint64_t* tmem_full_bar = empty_bar + kAgStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tma_a);
    for (int s = 0; s < 3; ++s) prefetch_tensormap(&tma_b.map[s]);
    for (int s = 0; s < kAgStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 8);  // 4 epilogue warps in each of the two CTAs
    }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, kTmemCols);
    tmem_relinquish<2>();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  tcgen05_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  const int m_blocks = (p.m_valid + kPairBM - 1) / kPairBM;
  const int num_items = plan.items;
  const int num_kb = p.k_blocks_per_seg * p.num_segs;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = cluster_id; i < num_items && ok; i += num_clusters) {
        int t, part, s, m_blk, n_blk;
        ag_item(i, plan, t, part, s);
        pair_tile_coords(t, p, m_blocks, m_blk, n_blk);
        const int a_row = m_blk * kPairBM + static_cast<int>(rank) * 128;
        const int b_share = 128 >> s;  // rows of B this CTA feeds to the pair's MMA
        const int b_row = n_blk * kBN + part * (kBN >> s) + static_cast<int>(rank) * b_share;
        const CUtensorMap* b_map = &tma_b.map[s];  // one load per stage: the box is the share
        const uint32_t tx = 2u * static_cast<uint32_t>(kPairABytes + b_share * kBK * 2);
        int seg = 0, kb_in_seg = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait<true>(&empty_bar[stage], phase ^ 1u, status, SILE_ERR_TIMEOUT, 1 + 4 * rank)) { ok = false; break; }
          uint8_t* sa = smem + stage * kPairStageBytes;
          uint8_t* sb = sa + kPairABytes;
          if (leader) mbar_expect_tx(&full_bar[stage], tx);
          tma_load_2d_pair(sa, &tma_a, &full_bar[stage], 0, kb_in_seg * kBK, p.a_seg_row[seg] + a_row);
          tma_load_2d_pair(sb, b_map, &full_bar[stage], 0, kb_in_seg * kBK, p.b_seg_row[seg] + b_row);
          if (++kb_in_seg == p.k_blocks_per_seg) { kb_in_seg = 0; ++seg; }
          if (++stage == kAgStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader) {
      const uint32_t el = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int i = cluster_id; i < num_items && ok; i += num_clusters, ++it) {
        int t, part, s;
        ag_item(i, plan, t, part, s);
        const uint32_t idesc = plan.idesc[s];
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait<true>(&tmem_empty_bar[buf], acc_phase ^ 1u, status, SILE_ERR_TIMEOUT, 2))) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait<true>(&full_bar[stage], phase, status, SILE_ERR_TIMEOUT, 3))) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kPairStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sa + kPairABytes, 16, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) umma_ss_f16_if<2>(el, tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_if<2>(el, pair_addr(&empty_bar[stage], 0));
          umma_commit_if<2>(el, pair_addr(&empty_bar[stage], 1));
          if (++stage == kAgStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          umma_commit_if<2>(el, pair_addr(&tmem_full_bar[buf], 0));
          umma_commit_if<2>(el, pair_addr(&tmem_full_bar[buf], 1));
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (both CTAs) ----------------
    const int quarter = warp & 3;
    uint8_t* stage = staging + quarter * (2 * 4096);
    const uint32_t stage_addr = smem_u32(stage);
    int it = 0;
    uint32_t slot = 0;  // staging box in turn, across items
    bool ok = true;
    for (int i = cluster_id; i < num_items && ok; i += num_clusters, ++it) {
      int t, part, s, m_blk, n_blk;
      ag_item(i, plan, t, part, s);
      pair_tile_coords(t, p, m_blocks, m_blk, n_blk);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait<true>(&tmem_full_bar[buf], acc_phase, status, SILE_ERR_TIMEOUT, 4 + 4 * rank)) { ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row0 = m_blk * kPairBM + static_cast<int>(rank) * 128;
      const int row = row0 + quarter * 32 + lane;
      const int width = kBN >> s;
      const int col_base = n_blk * kBN + part * width;
      const bool tile_fast = vec_ok && !p.masked && (row0 + 128 <= p.m_valid) && (col_base + width <= p.n_valid);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBN;
      if (tile_fast && !p.accumulate) {
        // destinations in an order that rotates with the item, so the GPUs do not all send to
        // the same peer at the same moment
        const int d0 = (peers.first + i) % peers.count;
        const int boxes = width / kBoxCols;
#pragma unroll 1
        for (int b = 0; b < boxes; ++b, slot ^= 1u) {  // boxes of 128 bytes x 32 rows
          uint32_t r[32], r2[sizeof(OutT) == 2 ? 32 : 1];
          tmem_ld_32x32b_x32(taddr + b * kBoxCols, r);
          if constexpr (sizeof(OutT) == 2) tmem_ld_32x32b_x32(taddr + b * kBoxCols + 32, r2);
          tcgen05_wait_ld();
          if (b == boxes - 1) {
            // last read of this accumulator: hand tensor memory back before the stores are issued
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(&tmem_empty_bar[buf], 0);
          }
          // the stores issued from this slot two boxes ago must have been read out of it
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          // row `lane` of the box: eight 16-byte chunks, chunk j stored at position j ^ (lane & 7)
          const uint32_t row_addr = stage_addr + slot * 4096 + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t v0, v1, v2, v3;
            const uint32_t* src = (sizeof(OutT) == 4) ? (r + 4 * j) : (j < 4) ? (r + 8 * j) : (r2 + 8 * (j - 4));
            if constexpr (sizeof(OutT) == 4) {
              v0 = src[0]; v1 = src[1]; v2 = src[2]; v3 = src[3];
            } else if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
              v0 = pack_bf16x2(__uint_as_float(src[0]), __uint_as_float(src[1]));
              v1 = pack_bf16x2(__uint_as_float(src[2]), __uint_as_float(src[3]));
              v2 = pack_bf16x2(__uint_as_float(src[4]), __uint_as_float(src[5]));
              v3 = pack_bf16x2(__uint_as_float(src[6]), __uint_as_float(src[7]));
            } else {
              __half2 h0 = __floats2half2_rn(__uint_as_float(src[0]), __uint_as_float(src[1]));
              __half2 h1 = __floats2half2_rn(__uint_as_float(src[2]), __uint_as_float(src[3]));
              __half2 h2 = __floats2half2_rn(__uint_as_float(src[4]), __uint_as_float(src[5]));
              __half2 h3 = __floats2half2_rn(__uint_as_float(src[6]), __uint_as_float(src[7]));
              v0 = *reinterpret_cast<uint32_t*>(&h0); v1 = *reinterpret_cast<uint32_t*>(&h1);
              v2 = *reinterpret_cast<uint32_t*>(&h2); v3 = *reinterpret_cast<uint32_t*>(&h3);
            }
            const uint32_t dst = row_addr + ((j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v0), "r"(v1), "r"(v2), "r"(v3) : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            int d = d0;
            for (int q = 0; q < peers.count; ++q) {
              tma_store_2d(&out_maps.map[d], stage + slot * 4096, col_base + b * kBoxCols, row0 + quarter * 32);
              if (++d == peers.count) d = 0;
            }
            tma_store_commit();
          }
        }
      } else {
#pragma unroll 1
        for (int ch = 0; ch < width / 32; ++ch) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + ch * 32, r);
          tcgen05_wait_ld();
          if (col_base + ch * 32 < p.n_valid) {
            int d = peers.first;
            for (int q = 0; q < peers.count; ++q) {
              store_chunk<OutT>(static_cast<OutT*>(peers.ptr[d]), p, row, col_base + ch * 32, r, tile_fast);
              if (++d == peers.count) d = 0;
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(&tmem_empty_bar[buf], 0);
      }
    }
    if (lane == 0) tma_store_wait_all<0>();  // every store of this warp has been written out
    __syncwarp();
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    if (*reinterpret_cast<volatile int*>(status) != 0) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {
      }
    }
    tmem_dealloc<2>(tmem_base, kTmemCols);
  }
}

// ---- wide CTA-pair variant -----------------------------------------------------------
// Same pairing, but one pair owns a 256 x 512 tile: per 64-wide k block each CTA stages its 128
// rows of A once and its 128-row shares of TWO 256-column B halves (48 KiB per stage, 4 stages),
// and the leader issues the k block's MMAs twice, once per half, into TMEM columns [0,256) and
// [256,512).  A is fetched from L2 once per 512 output columns instead of once per 256, which
// cuts L2 -> shared-memory traffic per flop by a quarter.  All 512 TMEM columns hold one tile, so
// the epilogue is not overlapped with the next tile's main loop (a few per cent of a tile once
// K reaches the thousands).  Eight epilogue warps: four per accumulator half.
constexpr int kWideStages = 4;
constexpr int kWideStageBytes = kPairABytes + 2 * kPairBBytes;
constexpr int kWideStagingBytes = 8 * 4096;  // one 32-row x 128-byte store box per epilogue warp
constexpr int kWideSmemBytes = kWideStages * kWideStageBytes + kWideStagingBytes + 256 + 1024;
constexpr int kWideBN = 512;
constexpr int kWideThreads = 320;

template <typename OutT>
__global__ void __launch_bounds__(kWideThreads, 1)
gemm_tn_pair_wide_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, OutT* __restrict__ c,
                         const GemmParams p, const uint32_t idesc, const int vec_ok, int* __restrict__ status,
                         const PeerOut peers, const __grid_constant__ OutMaps out_maps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + kWideStages * kWideStageBytes;  // 1024-byte aligned: matches the store maps' swizzle
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + kWideStagingBytes);
  uint64_t* empty_bar = full_bar + kWideStages;
  uint64_t* tmem_full_bar = empty_bar + kWideStages;   // [2]: one per accumulator half
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
    for (int s = 0; s < kWideStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(&tmem_full_bar[h], 1);
      mbar_init(&tmem_empty_bar[h], 8);  // 4 epilogue warps of this half in each of the two CTAs
    }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, kTmemCols);
    tmem_relinquish<2>();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  tcgen05_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  const int m_blocks = (p.m_valid + kPairBM - 1) / kPairBM;
  const int n_blocks = (p.n_valid + kWideBN - 1) / kWideBN;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = p.k_blocks_per_seg * p.num_segs;
  const int group = max(p.group_m / 2, 1);

  auto coords = [&](int t, int& m_blk, int& n_blk) {
    const int group_size = group * n_blocks;
    const int g = t / group_size;
    const int first_m = g * group;
    const int gm = min(m_blocks - first_m, group);
    const int r = t - g * group_size;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
  };

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int m_blk, n_blk;
        coords(t, m_blk, n_blk);
        const int a_row = m_blk * kPairBM + static_cast<int>(rank) * 128;
        const int b_row = n_blk * kWideBN + static_cast<int>(rank) * 128;
        int seg = 0, kb_in_seg = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait<true>(&empty_bar[stage], phase ^ 1u, status, SILE_ERR_TIMEOUT, 1 + 4 * rank)) { ok = false; break; }
          uint8_t* sa = smem + stage * kWideStageBytes;
          uint8_t* sb = sa + kPairABytes;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kWideStageBytes);
          const int x = kb_in_seg * kBK;
          tma_load_2d_pair(sa, &tma_a, &full_bar[stage], 0, x, p.a_seg_row[seg] + a_row);
          tma_load_2d_pair(sb, &tma_b, &full_bar[stage], 0, x, p.b_seg_row[seg] + b_row);
          tma_load_2d_pair(sb + kPairBBytes, &tma_b, &full_bar[stage], 0, x, p.b_seg_row[seg] + b_row + 256);
          if (++kb_in_seg == p.k_blocks_per_seg) { kb_in_seg = 0; ++seg; }
          if (++stage == kWideStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    // The whole warp runs the loop; the tcgen05 instructions are predicated on one elected lane
    // (see umma_ss_f16_if), which keeps descriptor arithmetic in the uniform datapath.
    if (leader) {
      const uint32_t el = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++it) {
        const uint32_t tile_phase = it & 1;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait<true>(&full_bar[stage], phase, status, SILE_ERR_TIMEOUT, 3))) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kWideStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (kb == 0) {
              // the previous tile's half h must have been drained by both CTAs' epilogue warps
              if (!__all_sync(0xffffffffu, mbar_wait<true>(&tmem_empty_bar[h], tile_phase ^ 1u, status, SILE_ERR_TIMEOUT, 2))) { ok = false; break; }
              tcgen05_fence_after();
            }
            const uint64_t bdesc = make_smem_desc_sw128(sa + kPairABytes + h * kPairBBytes, 16, 1024);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              umma_ss_f16_if<2>(el, tmem_base + h * 256, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            if (kb == num_kb - 1) {
              umma_commit_if<2>(el, pair_addr(&tmem_full_bar[h], 0));
              umma_commit_if<2>(el, pair_addr(&tmem_full_bar[h], 1));
            }
          }
          if (!ok) break;
          umma_commit_if<2>(el, pair_addr(&empty_bar[stage], 0));
          umma_commit_if<2>(el, pair_addr(&empty_bar[stage], 1));
          if (++stage == kWideStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (both CTAs; warps 2..5 drain half 0, warps 6..9 half 1) ----------------
    // Whole tiles go out through shared memory: each warp converts 32 rows x 128 bytes, writes
    // them in the 128-byte swizzle and lane 0 issues one TMA store per destination, so global
    // (and NVLink) writes are full 128-byte lines and the data movement needs no further
    // instructions.  TMEM is released as soon as the tile is in registers / staging, before the
    // stores drain.  Ragged or launch-masked tiles take the per-thread store path.
    const int quarter = warp & 3;
    const int h = (warp - 2) >> 2;
    constexpr int kBoxCols = 128 / static_cast<int>(sizeof(OutT));  // 64 (16-bit) or 32 (f32)
    uint8_t* stage = staging + (warp - 2) * 4096;
    const uint32_t stage_addr = smem_u32(stage);
    int it = 0;
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++it) {
      int m_blk, n_blk;
      coords(t, m_blk, n_blk);
      if (!mbar_wait<true>(&tmem_full_bar[h], it & 1, status, SILE_ERR_TIMEOUT, 4 + 4 * rank)) { ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int row0 = m_blk * kPairBM + static_cast<int>(rank) * 128;
      const int row = row0 + quarter * 32 + lane;
      const int col_base = n_blk * kWideBN + h * 256;
      const bool tile_fast = vec_ok && !p.masked && (row0 + 128 <= p.m_valid) && (col_base + 256 <= p.n_valid);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + h * 256;
      if (tile_fast && !p.accumulate) {
#pragma unroll 1
        for (int b = 0; b < 256 / kBoxCols; ++b) {
          uint32_t r[32], r2[32];
          tmem_ld_32x32b_x32(taddr + b * kBoxCols, r);
          if constexpr (kBoxCols == 64) tmem_ld_32x32b_x32(taddr + b * kBoxCols + 32, r2);
          tcgen05_wait_ld();
          if (b == 256 / kBoxCols - 1) {
            // last read of this accumulator half: hand TMEM back before the stores are issued
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(&tmem_empty_bar[h], 0);
          }
          if (lane == 0) tma_store_wait_read<0>();  // the previous box has left the staging buffer
          __syncwarp();
          // row `lane` of the box: eight 16-byte chunks, chunk j stored at position j ^ (lane & 7)
          const uint32_t row_addr = stage_addr + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t v0, v1, v2, v3;
            if constexpr (sizeof(OutT) == 4) {
              v0 = r[4 * j]; v1 = r[4 * j + 1]; v2 = r[4 * j + 2]; v3 = r[4 * j + 3];
            } else {
              const uint32_t* src = (j < 4) ? (r + 8 * j) : (r2 + 8 * (j - 4));
              if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
                v0 = pack_bf16x2(__uint_as_float(src[0]), __uint_as_float(src[1]));
                v1 = pack_bf16x2(__uint_as_float(src[2]), __uint_as_float(src[3]));
                v2 = pack_bf16x2(__uint_as_float(src[4]), __uint_as_float(src[5]));
                v3 = pack_bf16x2(__uint_as_float(src[6]), __uint_as_float(src[7]));
              } else {
                __half2 h0 = __floats2half2_rn(__uint_as_float(src[0]), __uint_as_float(src[1]));
                __half2 h1 = __floats2half2_rn(__uint_as_float(src[2]), __uint_as_float(src[3]));
                __half2 h2 = __floats2half2_rn(__uint_as_float(src[4]), __uint_as_float(src[5]));
                __half2 h3 = __floats2half2_rn(__uint_as_float(src[6]), __uint_as_float(src[7]));
                v0 = *reinterpret_cast<uint32_t*>(&h0); v1 = *reinterpret_cast<uint32_t*>(&h1);
                v2 = *reinterpret_cast<uint32_t*>(&h2); v3 = *reinterpret_cast<uint32_t*>(&h3);
              }
            }
            const uint32_t dst = row_addr + ((j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v0), "r"(v1), "r"(v2), "r"(v3) : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            int d = peers.first;
            for (int i = 0; i < peers.count; ++i) {
              tma_store_2d(&out_maps.map[d], stage, col_base + b * kBoxCols, row0 + quarter * 32);
              if (++d == peers.count) d = 0;
            }
            tma_store_commit();
          }
        }
      } else {
#pragma unroll 1
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + ch * 32, r);
          tcgen05_wait_ld();
          if (col_base + ch * 32 < p.n_valid) {
            int d = peers.first;
            for (int i = 0; i < peers.count; ++i) {
              store_chunk<OutT>(static_cast<OutT*>(peers.ptr[d]), p, row, col_base + ch * 32, r, tile_fast);
              if (++d == peers.count) d = 0;
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(&tmem_empty_bar[h], 0);
      }
    }
    if (lane == 0) tma_store_wait_all<0>();  // every store of this warp has been written out
    __syncwarp();
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    if (*reinterpret_cast<volatile int*>(status) != 0) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {
      }
    }
    tmem_dealloc<2>(tmem_base, kTmemCols);
  }
}

// ---- f32 -> (hi, lo) bf16 split pre-pass -----------------------------------------
// A: [M,K] f32 row-major -> hi/lo [M,Kp] bf16, zero for k >= k_eff.
__global__ void split_rows_kernel(const float* __restrict__ src, int64_t ld, __nv_bfloat16* __restrict__ hi,
                                  __nv_bfloat16* __restrict__ lo, int rows, int k_eff, int kp, int vec4) {
  const int groups_per_row = kp >> 3;
  const int64_t total = static_cast<int64_t>(rows) * groups_per_row;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(idx / groups_per_row);
    const int k0 = static_cast<int>(idx % groups_per_row) << 3;
    float x[8];
    const float* s = src + static_cast<int64_t>(row) * ld + k0;
    if (vec4 && k0 + 8 <= k_eff) {
      const float4 v0 = __ldg(reinterpret_cast<const float4*>(s));
      const float4 v1 = __ldg(reinterpret_cast<const float4*>(s) + 1);
      x[0] = v0.x; x[1] = v0.y; x[2] = v0.z; x[3] = v0.w;
      x[4] = v1.x; x[5] = v1.y; x[6] = v1.z; x[7] = v1.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = (k0 + i < k_eff) ? __ldg(s + i) : 0.0f;
    }
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat16 h0 = __float2bfloat16_rn(x[2 * i]);
      const __nv_bfloat16 h1 = __float2bfloat16_rn(x[2 * i + 1]);
      const float r0 = x[2 * i] - __bfloat162float(h0);
      const float r1 = x[2 * i + 1] - __bfloat162float(h1);
      h[i] = static_cast<uint32_t>(__bfloat16_as_ushort(h0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h1)) << 16);
      l[i] = pack_bf16x2(r0, r1);
    }
    const int64_t o = static_cast<int64_t>(row) * kp + k0;
    *reinterpret_cast<uint4*>(hi + o) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(lo + o) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

// B: [K,N] f32 row-major -> hi/lo [N,Kp] bf16 (transposed to K-major), zero for k >= k_eff.
// Block = 32 x 8 threads, tile = 64 (k) x 64 (n).  Reads run along n, 8 bytes per thread and 256
// bytes per warp and k row, eight rows in flight per thread; after the transpose through shared
// memory a thread owns 8 consecutive k of one n and writes them as one 16-byte store per plane,
// eight threads covering the tile's 128 bytes of a row.
__global__ void split_transpose_kernel(const float* __restrict__ src, int64_t ld, __nv_bfloat16* __restrict__ hi,
                                       __nv_bfloat16* __restrict__ lo, int n, int k_eff, int kp, int vec2) {
  __shared__ float tile[64][65];
  const int n0 = blockIdx.x * 64;
  const int k0 = blockIdx.y * 64;
  const int tx = threadIdx.x, ty = threadIdx.y;
  float2 v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int k = k0 + ty + 8 * i, col = n0 + 2 * tx;
    const float* s = src + static_cast<int64_t>(k) * ld + col;
    if (k < k_eff && vec2 && col + 1 < n) {
      v[i] = __ldg(reinterpret_cast<const float2*>(s));
    } else {
      v[i].x = (k < k_eff && col < n) ? __ldg(s) : 0.0f;
      v[i].y = (k < k_eff && col + 1 < n) ? __ldg(s + 1) : 0.0f;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    tile[ty + 8 * i][2 * tx] = v[i].x;
    tile[ty + 8 * i][2 * tx + 1] = v[i].y;
  }
  __syncthreads();
  const int kc = (tx & 7) * 8;  // first of this thread's 8 k values
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int nn = half * 32 + ty * 4 + (tx >> 3);  // row of the transposed tile
    const int col = n0 + nn;
    if (col < n) {
      uint32_t h[4], l[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float x0 = tile[kc + 2 * i][nn], x1 = tile[kc + 2 * i + 1][nn];
        const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
        h[i] = static_cast<uint32_t>(__bfloat16_as_ushort(h0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h1)) << 16);
        l[i] = pack_bf16x2(x0 - __bfloat162float(h0), x1 - __bfloat162float(h1));
      }
      const int64_t o = static_cast<int64_t>(col) * kp + k0 + kc;
      *reinterpret_cast<uint4*>(hi + o) = make_uint4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<uint4*>(lo + o) = make_uint4(l[0], l[1], l[2], l[3]);
    }
  }
}

// 16-bit B given row-major [K,N] -> [N,Kp] (K-major) so the same mainloop serves it.
template <typename T>
__global__ void transpose16_kernel(const T* __restrict__ src, int64_t ld, T* __restrict__ dst, int n, int k_eff, int kp) {
  __shared__ uint16_t tile[64][34];
  const int n0 = blockIdx.x * 32;
  const int k0 = blockIdx.y * 64;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
#pragma unroll
  for (int kk = ty; kk < 64; kk += 8) {
    const int k = k0 + kk, col = n0 + tx;
    tile[kk][tx] = (k < k_eff && col < n) ? s[static_cast<int64_t>(k) * ld + col] : static_cast<uint16_t>(0);
  }
  __syncthreads();
#pragma unroll
  for (int nn = ty; nn < 32; nn += 8) {
    const int col = n0 + nn;
    if (col < n) {
      const uint32_t v = static_cast<uint32_t>(tile[2 * tx][nn]) | (static_cast<uint32_t>(tile[2 * tx + 1][nn]) << 16);
      *reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(dst) + static_cast<int64_t>(col) * kp + k0 + 2 * tx) = v;
    }
  }
}

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

struct EffectiveDims {
  int64_t m_valid, n_valid, k_eff, kp;
};

EffectiveDims effective_dims(const GemmProblem& p) {
  EffectiveDims e;
  const int64_t bm = p.bm > 0 ? p.bm : 1, bn = p.bn > 0 ? p.bn : 1, bk = p.bk > 0 ? p.bk : 1;
  e.m_valid = p.m / bm * bm;
  e.n_valid = p.n / bn * bn;
  e.k_eff = p.k / bk * bk;
  e.kp = round_up(e.k_eff > 0 ? e.k_eff : 1, kBK);
  return e;
}

template <typename OutT>
int launch_typed(const CUtensorMap& ta, const CUtensorMap& tb, void* c, const GemmParams& gp, uint32_t idesc, int vec_ok,
                 int* status, int grid, cudaStream_t stream) {
  static bool attr_set[kMaxDevices] = {};  // per OutT instantiation and device
  if (!attr_set[current_device_slot()]) {
    SILE_CUDA_TRY(cudaFuncSetAttribute(gemm_tn_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set[current_device_slot()] = true;
  }
  gemm_tn_kernel<OutT><<<grid, kNumThreads, kSmemBytes, stream>>>(ta, tb, static_cast<OutT*>(c), gp, idesc, vec_ok, status);
  SILE_CUDA_TRY(cudaGetLastError());
  note_kernel(sizeof(OutT) == 4 ? "gemm_tn_kernel<f32>" : "gemm_tn_kernel<16-bit>", grid, kNumThreads, kSmemBytes);
  return SILE_OK;
}

template <typename OutT, bool kWide>
struct PairKernel {
  static auto fn() {
    if constexpr (kWide) return &gemm_tn_pair_wide_kernel<OutT>;
    else return &gemm_tn_pair_kernel<OutT>;
  }
  static constexpr int threads = kWide ? kWideThreads : kNumThreads;
  static constexpr int smem = kWide ? kWideSmemBytes : kPairSmemBytes;
  static constexpr int bn = kWide ? kWideBN : kBN;
};

template <typename OutT, bool kWide>
void pair_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int clusters, cudaStream_t stream) {
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg->gridDim = dim3(2 * clusters);
  cfg->blockDim = dim3(PairKernel<OutT, kWide>::threads);
  cfg->dynamicSmemBytes = PairKernel<OutT, kWide>::smem;
  cfg->stream = stream;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
}

// Number of 2-CTA clusters of a pair kernel that can be resident at once (0 = clusters cannot
// be scheduled on this device).  Queried once per kernel instantiation and device.
template <typename OutT, bool kWide>
int pair_max_clusters() {
  static int cache[kMaxDevices];
  static bool known[kMaxDevices] = {};
  const int slot = current_device_slot();
  if (known[slot]) return cache[slot];
  known[slot] = true;
  int& max_clusters = cache[slot];
  auto fn = PairKernel<OutT, kWide>::fn();
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, PairKernel<OutT, kWide>::smem) != cudaSuccess) {
    cudaGetLastError();
    return max_clusters = 0;
  }
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  pair_config<OutT, kWide>(&cfg, attr, sms / 2, nullptr);
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  return max_clusters = n;
}

template <bool kWide>
int pair_max_clusters_for(int out_dtype) {
  switch (out_dtype) {
    case SILE_DTYPE_F32: return pair_max_clusters<float, kWide>();
    case SILE_DTYPE_BF16: return pair_max_clusters<__nv_bfloat16, kWide>();
    default: return pair_max_clusters<__half, kWide>();
  }
}

template <typename OutT, bool kWide>
int launch_pair_typed(const CUtensorMap& ta, const CUtensorMap& tb, void* c, const GemmParams& gp, uint32_t idesc, int vec_ok,
                      int* status, cudaStream_t stream, const PeerOut& peers, const OutMaps* out_maps) {
  const int m_blocks = (gp.m_valid + kPairBM - 1) / kPairBM;
  const int n_blocks = (gp.n_valid + PairKernel<OutT, kWide>::bn - 1) / PairKernel<OutT, kWide>::bn;
  const int tiles = m_blocks * n_blocks;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  pair_config<OutT, kWide>(&cfg, attr, std::min(tiles, pair_max_clusters<OutT, kWide>()), stream);
  if constexpr (kWide) {
    SILE_CUDA_TRY(cudaLaunchKernelEx(&cfg, PairKernel<OutT, kWide>::fn(), ta, tb, static_cast<OutT*>(c), gp, idesc, vec_ok, status, peers,
                                     *out_maps));
  } else {
    SILE_CUDA_TRY(cudaLaunchKernelEx(&cfg, PairKernel<OutT, kWide>::fn(), ta, tb, static_cast<OutT*>(c), gp, idesc, vec_ok, status));
  }
  note_kernel(kWide ? (sizeof(OutT) == 4 ? "gemm_tn_pair_wide_kernel<f32>" : "gemm_tn_pair_wide_kernel<16-bit>")
                    : (sizeof(OutT) == 4 ? "gemm_tn_pair_kernel<f32>" : "gemm_tn_pair_kernel<16-bit>"),
              cfg.gridDim.x, cfg.blockDim.x, cfg.dynamicSmemBytes);
  return SILE_OK;
}

template <bool kWide>
int launch_pair(int out_dtype, const CUtensorMap& ta, const CUtensorMap& tb, void* c, const GemmParams& gp, uint32_t idesc, int vec_ok,
                int* status, cudaStream_t stream, const PeerOut& peers, const OutMaps* out_maps) {
  switch (out_dtype) {
    case SILE_DTYPE_F32: return launch_pair_typed<float, kWide>(ta, tb, c, gp, idesc, vec_ok, status, stream, peers, out_maps);
    case SILE_DTYPE_BF16: return launch_pair_typed<__nv_bfloat16, kWide>(ta, tb, c, gp, idesc, vec_ok, status, stream, peers, out_maps);
    default: return launch_pair_typed<__half, kWide>(ta, tb, c, gp, idesc, vec_ok, status, stream, peers, out_maps);
  }
}

// The all-gather pair kernel: resident clusters (cached per device) and launch.
template <typename OutT>
int ag_max_clusters() {
  static int cache[kMaxDevices];
  static bool known[kMaxDevices] = {};
  const int slot = current_device_slot();
  if (known[slot]) return cache[slot];
  known[slot] = true;
  int& max_clusters = cache[slot];
  auto fn = &gemm_tn_pair_sliced_kernel<OutT>;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kAgSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return max_clusters = 0;
  }
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2 * (sms / 2));
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = kAgSmemBytes;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  return max_clusters = n;
}

// The cut of the last, partly filled wave (log2 of the slices per tile) and the time that wave
// then takes, in whole-tile times.  Measured on 8192 x N x 8192: a half slice runs at 0.7 and a
// quarter slice at 0.4 of a whole tile's rate (A is fetched again for every slice).
int ag_tail_cut(int rest, int clusters, double* tail_time) {
  const double cost[3] = {1.0, 1.4, 2.5};
  int cut = 0;
  double best = rest > 0 ? 1.0 : 0.0;
  for (int s = 1; s <= 2 && rest > 0; ++s) {
    const int waves = ((rest << s) + clusters - 1) / clusters;
    const double t = cost[s] * waves / (1 << s);
    if (t < best - 0.05) { best = t; cut = s; }
  }
  if (tail_time) *tail_time = best;
  return cut;
}

// Whole-tile times the sliced kernel needs for `tiles` 256 x 256 tiles on `clusters` CTA pairs.
double ag_waves(int64_t tiles, int clusters) {
  clusters = std::max(clusters, 1);
  double tail = 0.0;
  ag_tail_cut(static_cast<int>(tiles % clusters), clusters, &tail);
  return static_cast<double>(tiles / clusters) + tail;
}

// Whole-tile times until the busiest CTA pair has finished its items of `plan` (item i runs on
// pair i mod clusters; a half slice costs 0.7 and a quarter 0.625 of a whole tile).
double ag_makespan(const AgPlan& plan, int clusters) {
  const double cost[3] = {1.0, 0.7, 0.625};
  clusters = std::max(clusters, 1);
  std::vector<double> busy(static_cast<size_t>(clusters), 0.0);
  int item = 0;
  for (int g = 0; g < plan.groups; ++g)
    for (int i = 0; i < (plan.n[g] << plan.s[g]); ++i, ++item) busy[static_cast<size_t>(item % clusters)] += cost[plan.s[g]];
  return *std::max_element(busy.begin(), busy.end());
}

// How the tiles are cut into work items.  Body: whole tiles.  Tail: when the last wave is partly
// filled, its tiles cut into the number of slices (2 or 4) that lets the clusters finish it
// soonest; slices run well below a whole tile's rate (more operand traffic per flop), which the
// estimate charges.  Head, with `stagger` (several destinations): a quarter wave of tiles cut in
// two, so half of the CTA pairs finish their first item after 0.7 of a tile time and stay 0.3 of a
// tile time ahead of the others; the waves' store bursts then reach NVLink in two halves
// (8192^3: 0.240 ms against 0.264 over 4 GPUs, 0.247 against 0.256 over 8; cutting a half wave,
// which leaves all pairs in step, was slower than no cut at all).  With `exchange_bound` as well
// (the peers' share of the output takes longer to cross NVLink than the tiles take to compute) the
// head puts the pairs into three phases instead (0.2405 ms over 8 GPUs).
// SILE_CUDA_GEMM_AG_SPLIT = off | s0,n0,s1,n1,...,s_last overrides it (tuning, tests): n0 tiles
// in 2^s0 slices, the next n1 in 2^s1, ..., the rest in 2^s_last; a negative n = the whole waves
// of what is left.
AgPlan make_ag_plan(int tiles, int clusters, bool bf16, bool stagger, bool exchange_bound) {
  AgPlan plan{};
  plan.idesc[0] = make_idesc_f16(kPairBM, kBN, bf16, false, false);
  plan.idesc[1] = make_idesc_f16(kPairBM, kBN / 2, bf16, false, false);
  plan.idesc[2] = make_idesc_f16(kPairBM, kBN / 4, bf16, false, false);
  clusters = std::max(clusters, 1);
  auto whole_waves = [&](int left) { return left / clusters * clusters; };
  int g = 0, left = tiles;
  auto add = [&](int n, int s) {
    n = std::min(std::max(n, 0), left);
    plan.n[g] = n; plan.s[g] = s;
    left -= n;
    ++g;
  };
  bool planned = false;
  if (const char* e = getenv("SILE_CUDA_GEMM_AG_SPLIT")) {
    if (!strcmp(e, "off")) {
      add(tiles, 0);
      planned = true;
    } else {
      long v[2 * kAgMaxGroups - 1];
      int count = 0;
      const char* c = e;
      while (count < 2 * kAgMaxGroups - 1) {
        char* end = nullptr;
        v[count] = strtol(c, &end, 10);
        if (end == c) break;
        ++count;
        if (*end != ',') break;
        c = end + 1;
      }
      bool ok = count % 2 == 1;
      for (int i = 0; ok && i < count; i += 2) ok = v[i] >= 0 && v[i] <= 2;
      if (ok) {
        for (int i = 0; i + 1 < count; i += 2) add(v[i + 1] < 0 ? whole_waves(left) : static_cast<int>(v[i + 1]), static_cast<int>(v[i]));
        add(left, static_cast<int>(v[count - 1]));
        planned = true;
      }
    }
  }
  if (!planned && stagger && exchange_bound && tiles > clusters) {
    // Three phases: two thirds of the pairs start with a half tile, half of those follow it with
    // a second one, the last third starts with a whole tile; first stores after 0.7, 1.0 and 1.4
    // tile times.  Whole tiles after that (the tail's cut does not matter: compute is not the bound).
    const int h1 = clusters / 3;
    add(h1, 1);
    add(clusters - 2 * h1, 0);
    add(h1 / 2, 1);
    add(left, 0);
    planned = true;
  }
  if (!planned) {
    if (stagger && tiles > clusters) add(clusters / 4, 1);
    add(whole_waves(left), 0);
    // The tail's cut: the one with which the busiest pair finishes soonest (the head may have
    // shifted the tail off a wave boundary); when the exchange bounds the step (here: fewer tiles
    // than CTA pairs), as fine as one wave allows, for smaller last stores.
    int cut = ag_tail_cut(left, clusters, nullptr);
    if (!exchange_bound && left > 0) {
      double best = 0.0;
      for (int c = 0; c <= 2; ++c) {
        AgPlan trial = plan;
        trial.n[g] = left; trial.s[g] = c; trial.groups = g + 1;
        const double t = ag_makespan(trial, clusters);
        if (c == 0 || t < best - 0.01) { best = t; cut = c; }
      }
    }
    add(left, cut);
  }
  plan.groups = g;
  plan.items = 0;
  for (int i = 0; i < g; ++i) plan.items += plan.n[i] << plan.s[i];
  return plan;
}

// The plan a launch would take, as text ("18x2+222x1+16x2": tiles x slices per tile, group by
// group), without launching anything.
AgPlan choose_ag_plan(int tiles, int clusters, bool bf16, int destinations, bool exchange_bound) {
  AgPlan plan = make_ag_plan(tiles, clusters, bf16, false, false);
  if (destinations > 1) {
    const AgPlan staggered = make_ag_plan(tiles, clusters, bf16, true, exchange_bound);
    if (exchange_bound || ag_makespan(staggered, clusters) <= 1.01 * ag_makespan(plan, clusters)) plan = staggered;
  }
  return plan;
}

int format_ag_plan(const AgPlan& plan, char* out, size_t cap) {
  int len = 0;
  if (cap > 0) out[0] = 0;
  for (int g = 0; g < plan.groups && len < static_cast<int>(cap) - 16; ++g)
    len += snprintf(out + len, cap - len, "%s%dx%d", g ? "+" : "", plan.n[g], 1 << plan.s[g]);
  return len;
}

template <typename OutT>
int launch_pair_ag(const CUtensorMap& ta, const AgBMaps& tb, const GemmParams& gp, bool bf16, int vec_ok, int* status,
                   cudaStream_t stream, const PeerOut& peers, const OutMaps& out_maps) {
  const int m_blocks = (gp.m_valid + kPairBM - 1) / kPairBM;
  const int tiles = m_blocks * gp.n_blocks;
  const int max_clusters = ag_max_clusters<OutT>();
  // Several destinations: the staggered head, unless it makes the busiest CTA pair finish later
  // and the exchange is not what bounds the step anyway (rates measured for this kernel on 8192^3
  // over 4 and 8 GPUs: 0.58 TB/s of peer stores leaving a GPU, 1.4 PFLOP/s of tensor work).
  const double k_total = static_cast<double>(gp.k_blocks_per_seg) * gp.num_segs * kBK;
  const double out_elems = static_cast<double>(gp.m_valid) * gp.n_valid;
  const double link_s = out_elems * sizeof(OutT) * (peers.count - 1) / 0.58e12;
  const double math_s = 2.0 * out_elems * k_total / 1.4e15;
  const AgPlan plan = choose_ag_plan(tiles, max_clusters, bf16, peers.count, link_s > math_s);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2 * std::min(plan.items, max_clusters));
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = kAgSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SILE_CUDA_TRY(cudaLaunchKernelEx(&cfg, &gemm_tn_pair_sliced_kernel<OutT>, ta, tb, gp, plan, vec_ok, status, peers, out_maps));
  // name, then the plan: tiles x slices per group, e.g. "plan=18x2+222x1+16x2"
  char name[160];
  const int len = snprintf(name, sizeof(name), "%s plan=", sizeof(OutT) == 4 ? "gemm_tn_pair_sliced_kernel<float>" : "gemm_tn_pair_sliced_kernel<16-bit>");
  format_ag_plan(plan, name + len, sizeof(name) - len);
  note_kernel(name, cfg.gridDim.x, cfg.blockDim.x, cfg.dynamicSmemBytes);
  return SILE_OK;
}

// SILE_CUDA_GEMM_AG_KERNEL = wide | pair picks the kernel of the fused GEMM + all-gather (tuning).
int forced_ag_kernel() {
  const char* e = getenv("SILE_CUDA_GEMM_AG_KERNEL");
  if (!e) return 0;
  if (!strcmp(e, "wide")) return 1;
  if (!strcmp(e, "pair")) return 2;
  return 0;
}

// SILE_CUDA_GEMM_KERNEL = single | pair | wide overrides the kernel choice (tuning, tests).
// Read on every launch so a process can switch.
int forced_kernel() {
  const char* e = getenv("SILE_CUDA_GEMM_KERNEL");
  if (!e) return 0;
  if (!strcmp(e, "single")) return 1;
  if (!strcmp(e, "pair")) return 2;
  if (!strcmp(e, "wide")) return 3;
  if (!strcmp(e, "sliced")) return 4;
  return 0;
}

// 128-row blocks per raster group (SILE_CUDA_GEMM_GROUP_M overrides, for tuning).
int raster_group_m(int fallback) {
  static const int g = [] {
    const char* e = getenv("SILE_CUDA_GEMM_GROUP_M");
    const int v = e ? atoi(e) : 0;
    return v > 0 ? v : 0;
  }();
  return g > 0 ? g : fallback;
}

}  // namespace

size_t gemm_workspace_bytes(const GemmProblem& p) {
  const EffectiveDims e = effective_dims(p);
  if (p.in_dtype == SILE_DTYPE_F32) {
    // hi and lo planes of A [M,Kp] and of B^T [N,Kp]
    return static_cast<size_t>(2 * (p.m + p.n) * e.kp) * sizeof(__nv_bfloat16);
  }
  if (p.b_layout == SILE_LAYOUT_ROW_MAJOR) return static_cast<size_t>(p.n * e.kp) * 2;  // B^T
  return 0;
}

int gemm_slice_plan_text(int tiles, int clusters, int destinations, int exchange_bound, char* out, size_t cap) {
  if (tiles <= 0 || clusters <= 0 || destinations < 1 || !out || cap < 32) return fail(SILE_ERR_INVALID, "slice plan: bad argument");
  format_ag_plan(choose_ag_plan(tiles, clusters, true, destinations, exchange_bound != 0), out, cap);
  return SILE_OK;
}

int gemm_launch(const GemmProblem& p, cudaStream_t stream) {
  if (!p.a || !p.b || !p.c) return fail(SILE_ERR_INVALID, "matmul: null buffer");
  if (p.m <= 0 || p.n <= 0 || p.k <= 0) return fail(SILE_ERR_INVALID, "matmul: non-positive dimension");
  if (p.m > (1ll << 30) || p.n > (1ll << 30) || p.k > (1ll << 30)) return fail(SILE_ERR_INVALID, "matmul: dimension too large");
  if (p.in_dtype != SILE_DTYPE_F32 && p.in_dtype != SILE_DTYPE_BF16 && p.in_dtype != SILE_DTYPE_F16)
    return fail(SILE_ERR_UNSUPPORTED, "matmul: unsupported input dtype %d", p.in_dtype);
  if (p.out_dtype != SILE_DTYPE_F32 && p.out_dtype != SILE_DTYPE_BF16 && p.out_dtype != SILE_DTYPE_F16)
    return fail(SILE_ERR_UNSUPPORTED, "matmul: unsupported output dtype %d", p.out_dtype);
  if (p.in_dtype == SILE_DTYPE_F32 && p.b_layout != SILE_LAYOUT_ROW_MAJOR)
    return fail(SILE_ERR_UNSUPPORTED, "matmul: f32 inputs are row-major only, as in the reference");

  const EffectiveDims e = effective_dims(p);
  const int64_t bm = p.bm > 0 ? p.bm : 1, bn = p.bn > 0 ? p.bn : 1;
  if (e.m_valid == 0 || e.n_valid == 0 || p.num_threadgroups <= 0) return SILE_OK;  // no whole tile launched

  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;

  const size_t need = gemm_workspace_bytes(p);
  if (need > 0 && (!p.workspace || p.workspace_bytes < need))
    return fail(SILE_ERR_INVALID, "matmul: workspace of %zu bytes required, %zu given", need, p.workspace_bytes);

  GemmParams gp{};
  gp.m_valid = static_cast<int>(e.m_valid);
  gp.n_valid = static_cast<int>(e.n_valid);
  gp.ldc = p.ldc > 0 ? p.ldc : p.n;
  if (gp.ldc < p.n) return fail(SILE_ERR_INVALID, "matmul: ldc smaller than N");
  gp.m_blocks = static_cast<int>((e.m_valid + kBM - 1) / kBM);
  gp.n_blocks = static_cast<int>((e.n_valid + kBN - 1) / kBN);
  gp.lbm = static_cast<int>(bm);
  gp.lbn = static_cast<int>(bn);
  gp.ltiles_n = static_cast<int>(p.n / bn);
  const long long total_logical = static_cast<long long>(p.m / bm) * (p.n / bn);
  gp.ntg = p.num_threadgroups;
  gp.masked = p.num_threadgroups < total_logical ? 1 : 0;
  gp.group_m = raster_group_m(kGroupM);
  gp.accumulate = p.accumulate ? 1 : 0;
  if (p.accumulate && p.num_peers > 0) return fail(SILE_ERR_UNSUPPORTED, "matmul: a seeded accumulator cannot be combined with the fused all-gather");

  CUtensorMap ta, tb;
  const bool bf16 = p.in_dtype != SILE_DTYPE_F16;
  const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  // Kernel choice, from measurements on 1024^3 .. 8192^3 problems: the wide pair kernel
  // (256 x 512 tiles) wins whenever it has enough tiles to occupy most of the 74 SM pairs; with
  // at most 256 output columns the 256 x 256 pair kernel takes its place; small problems keep
  // the single-CTA kernel, whose 128 x 256 tiles spread over more SMs.  In a pair each CTA
  // stages 128-row boxes of B, so the B box differs from the single-CTA kernel's.
  const int forced = forced_kernel();
  const int64_t tiles_pair = ((e.m_valid + kPairBM - 1) / kPairBM) * ((e.n_valid + kBN - 1) / kBN);
  const int64_t tiles_wide = ((e.m_valid + kPairBM - 1) / kPairBM) * ((e.n_valid + kWideBN - 1) / kWideBN);
  constexpr int64_t kMinPairTiles = 48;
  bool use_wide = false, use_pair = false;
  if (forced == 3 || p.num_peers > 0 || (forced == 0 && e.n_valid > kBN && tiles_wide >= kMinPairTiles)) {
    use_wide = e.m_valid > kBM && pair_max_clusters_for<true>(p.out_dtype) > 0;
  } else if (forced == 2 || (forced == 0 && e.n_valid <= kBN && tiles_pair >= kMinPairTiles)) {
    use_pair = e.m_valid > kBM && pair_max_clusters_for<false>(p.out_dtype) > 0;
  }
  // Fused GEMM + all-gather: the 256 x 256 pair kernel whose epilogue stages whole tiles and lets
  // the stores to every destination drain under the following tiles (16-bit outputs); the wide
  // kernel otherwise, or when asked for.
  // One GPU: the sliced kernel instead of the wide one when its 256 x 256 tiles fill the CTA pairs'
  // waves better (8192 x 4096 x 8192: 6.9 waves against 3.46 -> 4 of the wide tiles, 0.333 ms
  // against 0.366); per flop in a full wave the wide kernel is 3 % ahead.
  bool prefer_sliced = false;
  if (forced == 0 && p.num_peers == 0 && use_wide) {
    const int clusters = p.out_dtype == SILE_DTYPE_F32    ? ag_max_clusters<float>()
                         : p.out_dtype == SILE_DTYPE_BF16 ? ag_max_clusters<__nv_bfloat16>()
                                                          : ag_max_clusters<__half>();
    const int wide_clusters = pair_max_clusters_for<true>(p.out_dtype);
    if (clusters > 0 && wide_clusters > 0) {
      const double wide_time = 2.0 * static_cast<double>((tiles_wide + wide_clusters - 1) / wide_clusters) / 1.03;
      prefer_sliced = ag_waves(tiles_pair, clusters) < 0.96 * wide_time;
    }
  }
  bool use_ag = false;
  if (e.m_valid > kBM && ((p.num_peers > 0 && forced_ag_kernel() != 1) || (p.num_peers == 0 && (forced == 4 || prefer_sliced)))) {
    use_ag = (p.out_dtype == SILE_DTYPE_F32    ? ag_max_clusters<float>()
              : p.out_dtype == SILE_DTYPE_BF16 ? ag_max_clusters<__nv_bfloat16>()
                                               : ag_max_clusters<__half>()) > 0;
    if (use_ag) use_wide = false;
  }
  use_pair = use_pair || use_wide || use_ag;
  // The wide kernel's raster groups are twice as tall (32 blocks of 128 rows): 8192^3 under
  // sustained load 1553 against 1541 TFLOP/s (24 blocks: 1548).
  if (use_wide) gp.group_m = raster_group_m(2 * kGroupM);
  const uint32_t box_a[2] = {kBK, kBM};
  const uint32_t box_b[2] = {kBK, use_pair ? 128u : static_cast<uint32_t>(kBN)};
  static const AgBMaps zero_b_maps{};
  AgBMaps tb_ag = zero_b_maps;  // the sliced kernel's three maps of B

  if (p.in_dtype == SILE_DTYPE_F32) {
    if (e.k_eff == 0) {
      // Zero-trip k loop: the reference stores the 0.0f accumulator.  Same code path, all-zero operands.
    }
    auto* ws = static_cast<__nv_bfloat16*>(p.workspace);
    __nv_bfloat16* a_hi = ws;
    __nv_bfloat16* a_lo = a_hi + p.m * e.kp;
    __nv_bfloat16* b_hi = a_lo + p.m * e.kp;
    __nv_bfloat16* b_lo = b_hi + p.n * e.kp;
    {
      const int64_t total = p.m * (e.kp >> 3);
      const int threads = 256;
      const int blocks = static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 148 * 16));
      const int vec4 = (p.k % 4 == 0) && (reinterpret_cast<uintptr_t>(p.a) % 16 == 0);
      split_rows_kernel<<<blocks, threads, 0, stream>>>(static_cast<const float*>(p.a), p.k, a_hi, a_lo, static_cast<int>(p.m),
                                                        static_cast<int>(e.k_eff), static_cast<int>(e.kp), vec4);
      SILE_CUDA_TRY(cudaGetLastError());
    }
    {
      dim3 grid(static_cast<unsigned>((p.n + 63) / 64), static_cast<unsigned>(e.kp / 64));
      const int vec2 = (p.n % 2 == 0) && (reinterpret_cast<uintptr_t>(p.b) % 8 == 0);
      split_transpose_kernel<<<grid, dim3(32, 8), 0, stream>>>(static_cast<const float*>(p.b), p.n, b_hi, b_lo,
                                                               static_cast<int>(p.n), static_cast<int>(e.k_eff),
                                                               static_cast<int>(e.kp), vec2);
      SILE_CUDA_TRY(cudaGetLastError());
    }
    // Tensor maps over the stacked planes: rows [0,M) = hi, [M,2M) = lo.
    const uint64_t dims_a[2] = {static_cast<uint64_t>(e.kp), static_cast<uint64_t>(2 * p.m)};
    const uint64_t dims_b[2] = {static_cast<uint64_t>(e.kp), static_cast<uint64_t>(2 * p.n)};
    const uint64_t stride[1] = {static_cast<uint64_t>(e.kp) * 2};
    if (int rc = encode_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_hi, dims_a, stride, box_a, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    if (int rc = encode_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_hi, dims_b, stride, box_b, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    for (int s = 0; use_ag && s < 3; ++s) {
      const uint32_t box[2] = {kBK, 128u >> s};
      if (int rc = encode_tensor_map(&tb_ag.map[s], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_hi, dims_b, stride, box, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    }
    gp.num_segs = 3;
    gp.k_blocks_per_seg = static_cast<int>(e.kp / kBK);
    // small terms first: lo*hi, hi*lo, then hi*hi
    gp.a_seg_row[0] = static_cast<int>(p.m); gp.b_seg_row[0] = 0;
    gp.a_seg_row[1] = 0;                     gp.b_seg_row[1] = static_cast<int>(p.n);
    gp.a_seg_row[2] = 0;                     gp.b_seg_row[2] = 0;
  } else {
    if (p.k % 8 != 0 || reinterpret_cast<uintptr_t>(p.a) % 16 != 0 || reinterpret_cast<uintptr_t>(p.b) % 16 != 0)
      return fail(SILE_ERR_UNSUPPORTED, "matmul: 16-bit operands need K %% 8 == 0 and 16-byte aligned bases");
    if (e.k_eff == 0) return fail(SILE_ERR_UNSUPPORTED, "matmul: K smaller than BK with 16-bit operands");
    const void* b_kmajor = p.b;
    uint64_t b_ld = static_cast<uint64_t>(p.k);
    uint64_t b_kdim = static_cast<uint64_t>(e.k_eff);
    if (p.b_layout == SILE_LAYOUT_ROW_MAJOR) {
      dim3 grid(static_cast<unsigned>((p.n + 31) / 32), static_cast<unsigned>(e.kp / 64));
      transpose16_kernel<uint16_t><<<grid, dim3(32, 8), 0, stream>>>(static_cast<const uint16_t*>(p.b), p.n,
                                                                     static_cast<uint16_t*>(p.workspace), static_cast<int>(p.n),
                                                                     static_cast<int>(e.k_eff), static_cast<int>(e.kp));
      SILE_CUDA_TRY(cudaGetLastError());
      b_kmajor = p.workspace;
      b_ld = static_cast<uint64_t>(e.kp);
      b_kdim = static_cast<uint64_t>(e.kp);
    }
    // Inner extent k_eff: reads past it are zero-filled by TMA, which is how the
    // reference's dropped K remainder is honoured.
    const uint64_t dims_a[2] = {static_cast<uint64_t>(e.k_eff), static_cast<uint64_t>(p.m)};
    const uint64_t dims_b[2] = {b_kdim, static_cast<uint64_t>(p.n)};
    const uint64_t stride_a[1] = {static_cast<uint64_t>(p.k) * 2};
    const uint64_t stride_b[1] = {b_ld * 2};
    if (int rc = encode_tensor_map(&ta, dt, 2, p.a, dims_a, stride_a, box_a, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    if (int rc = encode_tensor_map(&tb, dt, 2, b_kmajor, dims_b, stride_b, box_b, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    for (int s = 0; use_ag && s < 3; ++s) {
      const uint32_t box[2] = {kBK, 128u >> s};
      if (int rc = encode_tensor_map(&tb_ag.map[s], dt, 2, b_kmajor, dims_b, stride_b, box, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    }
    gp.num_segs = 1;
    gp.k_blocks_per_seg = static_cast<int>((e.k_eff + kBK - 1) / kBK);
  }

  const size_t out_elt = p.out_dtype == SILE_DTYPE_F32 ? 4 : 2;
  const int vec_ok = (reinterpret_cast<uintptr_t>(p.c) % 16 == 0) && ((gp.ldc * out_elt) % 16 == 0);
  PeerOut peers{};
  if (p.num_peers > 0) {
    if (!use_wide && !use_ag) return fail(SILE_ERR_UNSUPPORTED, "matmul: the fused all-gather epilogue needs a CTA-pair kernel (M > 128)");
    for (int i = 0; i < p.num_peers; ++i) peers.ptr[i] = p.peer_c[i];
    peers.count = p.num_peers;
    peers.first = p.peer_first;
  } else {
    peers.ptr[0] = p.c;
    peers.count = 1;
    peers.first = 0;
  }
  if (use_pair) {
    const uint32_t idesc2 = make_idesc_f16(kPairBM, kBN, bf16, false, false);
    if (!use_wide && !use_ag) return launch_pair<false>(p.out_dtype, ta, tb, p.c, gp, idesc2, vec_ok, status, stream, peers, nullptr);
    static OutMaps zero_maps{};
    OutMaps maps = zero_maps;
    if (vec_ok) {
      // Store maps: columns from the block's first column to the end of the row (the kernel
      // only stores whole tiles inside the valid region through them), all M rows.
      const CUtensorMapDataType odt = p.out_dtype == SILE_DTYPE_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                    : p.out_dtype == SILE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
      const uint64_t odims[2] = {static_cast<uint64_t>(p.n), static_cast<uint64_t>(p.m)};
      const uint64_t ostride[1] = {static_cast<uint64_t>(gp.ldc) * out_elt};
      const uint32_t obox[2] = {static_cast<uint32_t>(128 / out_elt), 32};
      for (int i = 0; i < peers.count; ++i)
        if (int rc = encode_tensor_map(&maps.map[i], odt, 2, peers.ptr[i], odims, ostride, obox, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    }
    if (use_ag) {
      if (p.out_dtype == SILE_DTYPE_F32) return launch_pair_ag<float>(ta, tb_ag, gp, bf16, vec_ok, status, stream, peers, maps);
      if (p.out_dtype == SILE_DTYPE_BF16) return launch_pair_ag<__nv_bfloat16>(ta, tb_ag, gp, bf16, vec_ok, status, stream, peers, maps);
      return launch_pair_ag<__half>(ta, tb_ag, gp, bf16, vec_ok, status, stream, peers, maps);
    }
    return launch_pair<true>(p.out_dtype, ta, tb, p.c, gp, idesc2, vec_ok, status, stream, peers, &maps);
  }
  const uint32_t idesc = make_idesc_f16(kBM, kBN, bf16, false, false);
  const int num_tiles = gp.m_blocks * gp.n_blocks;
  int dev = 0, sms = 148;
  SILE_CUDA_TRY(cudaGetDevice(&dev));
  SILE_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int grid = std::min(num_tiles, sms);

  switch (p.out_dtype) {
    case SILE_DTYPE_F32: return launch_typed<float>(ta, tb, p.c, gp, idesc, vec_ok, status, grid, stream);
    case SILE_DTYPE_BF16: return launch_typed<__nv_bfloat16>(ta, tb, p.c, gp, idesc, vec_ok, status, grid, stream);
    default: return launch_typed<__half>(ta, tb, p.c, gp, idesc, vec_ok, status, grid, stream);
  }
}

}  // namespace sile

// ---- f32 matmul without any allocation ------------------------------------------------
// Some hosts cannot let a library allocate device memory: a serving process that has handed
// all of HBM to its own arena (a cudaMalloc there fails, or fragments the arena's neighbour),
// a control loop that must not take the driver's allocation lock or its implicit device-wide
// synchronisation, a deployment whose policy forbids allocation after start-up.  For them the
// scratch of the f32 split lives in a fixed array inside the library image and the time-out
// status word beside it; nothing below calls cudaMalloc, cudaMallocAsync, cudaFree or any
// allocating library routine.
//
// The array's name is only a host-side handle for the symbol: host code must never pass it to
// a kernel.  The device address is looked up with cudaGetSymbolAddress once per device, with
// that device current, and the kernels receive that pointer.
namespace sile {
namespace {

constexpr size_t kNoAllocScratchBytes = size_t(32) << 20;  // 32 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
static __device__ int g_noalloc_status;

struct NoAllocDevice {
  void* scratch = nullptr;
  int* status = nullptr;
};
NoAllocDevice g_noalloc_dev[64];
std::mutex g_noalloc_mutex;

// First use on a device: resolves the device addresses of the two symbols and raises the
// kernel's dynamic shared-memory limit.  Must run outside stream capture.
int noalloc_setup(int dev, NoAllocDevice* out) {
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoAllocDevice& d = g_noalloc_dev[dev];
  if (!d.scratch) {
    void* scratch = nullptr;
    void* status = nullptr;
    SILE_CUDA_TRY(cudaGetSymbolAddress(&scratch, g_noalloc_scratch));
    SILE_CUDA_TRY(cudaGetSymbolAddress(&status, g_noalloc_status));
    SILE_CUDA_TRY(cudaFuncSetAttribute(gemm_tn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    d.scratch = scratch;
    d.status = static_cast<int*>(status);
  }
  *out = d;
  return SILE_OK;
}

}  // namespace

int noalloc_read_and_clear_status(int* value) {
  *value = 0;
  int dev = 0;
  SILE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return SILE_OK;
  int* word = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    word = g_noalloc_dev[dev].status;
  }
  if (!word) return SILE_OK;  // the entry point has not run on this device
  SILE_CUDA_TRY(cudaMemcpy(value, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (*value != 0) SILE_CUDA_TRY(cudaMemset(word, 0, sizeof(int)));
  return SILE_OK;
}

}  // namespace sile

extern "C" int sile_cuda_matmul_f32_noalloc(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                                            int64_t bm, int64_t bn, int64_t bk, void* stream_handle, int32_t wait) {
  using namespace sile;
  if (!a || !b || !c) return fail(SILE_ERR_INVALID, "matmul_f32_noalloc: null buffer");
  if (m <= 0 || n <= 0 || k <= 0) return fail(SILE_ERR_INVALID, "matmul_f32_noalloc: non-positive dimension");
  if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return fail(SILE_ERR_INVALID, "matmul_f32_noalloc: dimension too large");
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return fail(SILE_ERR_NO_DEVICE, "matmul_f32_noalloc: no CUDA device");
  }
  int major = 0;
  SILE_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10 || dev < 0 || dev >= 64) return fail(SILE_ERR_NO_DEVICE, "matmul_f32_noalloc: device %d is not a usable sm_100 GPU", dev);

  GemmProblem p;
  p.a = a; p.b = b; p.c = c;
  p.m = m; p.n = n; p.k = k;
  p.bm = bm > 0 ? bm : 1; p.bn = bn > 0 ? bn : 1; p.bk = bk > 0 ? bk : 1;
  const EffectiveDims e = effective_dims(p);
  const size_t need = static_cast<size_t>(2 * (m + n) * e.kp) * sizeof(__nv_bfloat16);
  if (need > kNoAllocScratchBytes)
    return fail(SILE_ERR_UNSUPPORTED,
                "matmul_f32_noalloc: this problem needs %zu bytes of scratch (4 * (M + N) * K rounded up to 64); the built-in "
                "array holds %zu bytes -- use sile_cuda_launch for larger problems", need, kNoAllocScratchBytes);
  if (e.m_valid == 0 || e.n_valid == 0) return SILE_OK;  // no whole logical tile

  NoAllocDevice nd;
  if (int rc = noalloc_setup(dev, &nd)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);

  // Planes A_hi | A_lo ([2M, Kp]) then B^T_hi | B^T_lo ([2N, Kp]).  Both split kernels write
  // every element of their planes, zero padding included, so nothing left over from an earlier
  // call is ever read.
  auto* a_hi = static_cast<__nv_bfloat16*>(nd.scratch);
  __nv_bfloat16* a_lo = a_hi + m * e.kp;
  __nv_bfloat16* b_hi = a_lo + m * e.kp;
  __nv_bfloat16* b_lo = b_hi + n * e.kp;
  {
    const int64_t total = m * (e.kp >> 3);
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 148 * 16));
    const int vec4 = (k % 4 == 0) && (reinterpret_cast<uintptr_t>(a) % 16 == 0);
    split_rows_kernel<<<blocks, threads, 0, stream>>>(a, k, a_hi, a_lo, static_cast<int>(m), static_cast<int>(e.k_eff),
                                                      static_cast<int>(e.kp), vec4);
    SILE_CUDA_TRY(cudaGetLastError());
    dim3 grid(static_cast<unsigned>((n + 63) / 64), static_cast<unsigned>(e.kp / 64));
    const int vec2 = (n % 2 == 0) && (reinterpret_cast<uintptr_t>(b) % 8 == 0);
    split_transpose_kernel<<<grid, dim3(32, 8), 0, stream>>>(b, n, b_hi, b_lo, static_cast<int>(n), static_cast<int>(e.k_eff),
                                                             static_cast<int>(e.kp), vec2);
    SILE_CUDA_TRY(cudaGetLastError());
  }

  CUtensorMap ta, tb;
  const uint32_t box_a[2] = {kBK, kBM};
  const uint32_t box_b[2] = {kBK, kBN};
  const uint64_t dims_a[2] = {static_cast<uint64_t>(e.kp), static_cast<uint64_t>(2 * m)};
  const uint64_t dims_b[2] = {static_cast<uint64_t>(e.kp), static_cast<uint64_t>(2 * n)};
  const uint64_t stride[1] = {static_cast<uint64_t>(e.kp) * 2};
  if (int rc = encode_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_hi, dims_a, stride, box_a, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = encode_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_hi, dims_b, stride, box_b, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;

  GemmParams gp{};
  gp.m_valid = static_cast<int>(e.m_valid);
  gp.n_valid = static_cast<int>(e.n_valid);
  gp.ldc = n;
  gp.m_blocks = static_cast<int>((e.m_valid + kBM - 1) / kBM);
  gp.n_blocks = static_cast<int>((e.n_valid + kBN - 1) / kBN);
  gp.lbm = static_cast<int>(p.bm);
  gp.lbn = static_cast<int>(p.bn);
  gp.ltiles_n = static_cast<int>(n / p.bn);
  gp.ntg = INT64_MAX;
  gp.masked = 0;
  gp.group_m = kGroupM;
  gp.num_segs = 3;
  gp.k_blocks_per_seg = static_cast<int>(e.kp / kBK);
  gp.a_seg_row[0] = static_cast<int>(m); gp.b_seg_row[0] = 0;
  gp.a_seg_row[1] = 0;                   gp.b_seg_row[1] = static_cast<int>(n);
  gp.a_seg_row[2] = 0;                   gp.b_seg_row[2] = 0;

  int sms = 148;
  SILE_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int grid = std::min(gp.m_blocks * gp.n_blocks, sms);
  const int vec_ok = (reinterpret_cast<uintptr_t>(c) % 16 == 0) && ((n * 4) % 16 == 0);
  const uint32_t idesc = make_idesc_f16(kBM, kBN, true, false, false);
  gemm_tn_kernel<float><<<grid, kNumThreads, kSmemBytes, stream>>>(ta, tb, c, gp, idesc, vec_ok, nd.status);
  SILE_CUDA_TRY(cudaGetLastError());

  if (wait) {
    SILE_CUDA_TRY(cudaStreamSynchronize(stream));
    int st = 0;
    if (int rc = noalloc_read_and_clear_status(&st)) return rc;
    return decode_status_word(st);
  }
  return SILE_OK;
}
