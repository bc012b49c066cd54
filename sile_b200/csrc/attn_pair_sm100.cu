// Fused attention forward for sm_100a, CTA-pair form: the two CTAs of a cluster (two SMs) take
// 128 query rows each of one (batch, head) and SHARE every K / V block.
//
// Same algorithm and numerics as the single-CTA kernel in attn_sm100.cu (online softmax over
// 128-key blocks, f32 statistics, lazily rescaled accumulator).  What changes:
//   * the MMAs are tcgen05 cta_group::2 instructions issued by the leader CTA: S (256 x 128) =
//     [Q of CTA0; Q of CTA1] K^T takes the N = 128 keys half from each CTA's shared memory, and
//     O += P V takes the N = 128 head-dim columns half from each.  Of every K block each CTA
//     stages only its 64 keys, of every V block only its 64 head-dim columns, so the pair pulls
//     each K / V byte from L2 once per 256 query rows, like the single-CTA kernel, while each SM
//     holds ONE Q tile;
//   * with one tile per SM the 512 tensor-memory columns hold THREE S buffers next to O.  The
//     issue order S0 S1 S2 | PV0 S3 | PV1 S4 | ... puts Q K^T of block j+3 in flight as soon as
//     P_j has been consumed, so the softmax warps never wait for the tensor core: the step that
//     bounds the kernel, 128 exp2 per row and block on the 16-lane MUFU pipe, runs back to back
//     instead of alternating with the tile's own MMAs.
//
// No counterpart in the reference: attention there is a composition of tile ops
// (crates/sile-tile-ir/src/lower.rs:509-748), and the reference has no CUDA backend.
#include <cuda_bf16.h>

#include <algorithm>

#include "internal.h"
#include "ptx.cuh"

namespace sile {
namespace {

using namespace ptx;

constexpr int kD = 128;             // head dim
constexpr int kTileQ = 128;         // rows per CTA (= TMEM lanes)
constexpr int kPairQ = 2 * kTileQ;  // rows one cta_group::2 MMA covers
constexpr int kBlockKV = 128;
constexpr int kBufS = 3;            // S buffers in tensor memory
constexpr int kQPanelBytes = kTileQ * 64 * 2;       // [128 rows x 64 d], 128B-swizzled
constexpr int kQTileBytes = 2 * kQPanelBytes;       // [128 x 128]
constexpr int kKPanelBytes = (kBlockKV / 2) * 64 * 2;  // this CTA's [64 keys x 64 d]
constexpr int kKStageBytes = 2 * kKPanelBytes;         // [64 keys x 128 d]
constexpr int kVStageBytes = kBlockKV * 64 * 2;        // this CTA's [128 keys x 64 d]
constexpr int kStagesK = 5;  // S_{j+3} is issued while block j is still in its softmax
constexpr int kStagesV = 4;
constexpr int kThreads = 192;
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + kQTileBytes;
constexpr int kSmemV = kSmemK + kStagesK * kKStageBytes;
constexpr int kSmemBar = kSmemV + kStagesV * kVStageBytes;
constexpr int kSmemBytes = kSmemBar + 512 + 1024;
constexpr uint32_t kTmemCols = 512;  // S0 | S1 | S2 | O
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct PairParams {
  int s;            // sequence length
  int bh;           // batch * heads
  int num_qblocks;  // 256-row query blocks per head
  int causal;
  float scale_log2;    // scale * log2(e)
  int64_t row_stride;  // elements between consecutive rows of O (= D)
};

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));  // volatile: keeps the staged order below
  return y;
}

// Number of 128-key blocks the 256 query rows starting at q0 attend to.  Both CTAs of the pair
// run the same count: their MMAs are one instruction.
__device__ __forceinline__ int kv_blocks_for_rows(const PairParams& p, int q0) {
  const int all = (p.s + kBlockKV - 1) / kBlockKV;
  if (!p.causal) return all;
  const int last_q = min(q0 + kPairQ, p.s) - 1;
  return min(all, last_q / kBlockKV + 1);
}

__device__ __forceinline__ void commit_both(uint32_t elected, uint64_t* bar) {
  umma_commit_if<2>(elected, pair_addr(bar, 0));
  umma_commit_if<2>(elected, pair_addr(bar, 1));
}

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, __nv_bfloat16* __restrict__ o, const PairParams p,
                     int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  // Every barrier exists at the same offset in both CTAs.  Waited on in the LEADER only:
  // q_full, k_full, v_full (both CTAs' TMA loads complete on the leader's copy) and p_full.
  // Waited on locally in each CTA, signalled by the leader's commits: the rest.
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemBar);
  uint64_t* q_full = bars;                  // [1]
  uint64_t* k_full = q_full + 1;            // [kStagesK]
  uint64_t* k_empty = k_full + kStagesK;    // [kStagesK]
  uint64_t* v_full = k_empty + kStagesK;    // [kStagesV]
  uint64_t* v_empty = v_full + kStagesV;    // [kStagesV] V stage free = O += P_j V_j finished
  uint64_t* s_full = v_empty + kStagesV;    // [kBufS] S buffer written by the tensor core
  uint64_t* p_full = s_full + kBufS;        // [kBufS] P written over the S buffer (and O rescaled) by both CTAs' softmax warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_full + kBufS);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  // Cluster order: heads in groups of kHeadGroup; inside a group the late query blocks (heavy
  // under a causal mask) of every head come first, so resident clusters share a few heads' K / V
  // in L2 and the clusters that finish last are the light ones.
  constexpr int kHeadGroup = 8;
  const int cluster_id = blockIdx.x >> 1;
  const int group = cluster_id / (kHeadGroup * p.num_qblocks);
  const int in_group = cluster_id - group * kHeadGroup * p.num_qblocks;
  const int heads_here = min(kHeadGroup, p.bh - group * kHeadGroup);
  const int bh = group * kHeadGroup + in_group % heads_here;
  const int qblk = p.num_qblocks - 1 - in_group / heads_here;
  const int q_base = qblk * kPairQ;
  const int n = kv_blocks_for_rows(p, q_base);

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tma_q);
    prefetch_tensormap(&tma_k);
    prefetch_tensormap(&tma_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < kStagesK; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < kStagesV; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < kBufS; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 8);  // 4 softmax warps in each of the two CTAs
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
  const uint32_t tmem_s[kBufS] = {tmem_base, tmem_base + 128, tmem_base + 256};
  const uint32_t tmem_o = tmem_base + 384;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs; completions land on the leader's barriers) ----------------
    if (lane == 0 && n > 0) {
      bool ok = true;
      const int r = static_cast<int>(rank);
      {
        if (leader) mbar_expect_tx(q_full, 2 * kQTileBytes);
        const int row0 = q_base + r * kTileQ;
        tma_load_3d_pair(smem + kSmemQ, &tma_q, q_full, 0, 0, row0, bh);
        tma_load_3d_pair(smem + kSmemQ + kQPanelBytes, &tma_q, q_full, 0, 64, row0, bh);
      }
      for (int j = 0; j < n && ok; ++j) {
        const int sk = j % kStagesK, sv = j % kStagesV;
        // this CTA's 64 keys of block j, both head-dim panels
        if (!mbar_wait<true>(&k_empty[sk], ((j / kStagesK) & 1) ^ 1u, status, SILE_ERR_TIMEOUT, 1)) { ok = false; break; }
        if (leader) mbar_expect_tx(&k_full[sk], 2 * kKStageBytes);
        uint8_t* dk = smem + kSmemK + sk * kKStageBytes;
        const int krow = j * kBlockKV + r * (kBlockKV / 2);
        tma_load_3d_pair(dk, &tma_k, &k_full[sk], 0, 0, krow, bh);
        tma_load_3d_pair(dk + kKPanelBytes, &tma_k, &k_full[sk], 0, 64, krow, bh);
        // all 128 keys of block j, this CTA's 64 head-dim columns
        if (!mbar_wait<true>(&v_empty[sv], ((j / kStagesV) & 1) ^ 1u, status, SILE_ERR_TIMEOUT, 2)) { ok = false; break; }
        if (leader) mbar_expect_tx(&v_full[sv], 2 * kVStageBytes);
        tma_load_3d_pair(smem + kSmemV + sv * kVStageBytes, &tma_v, &v_full[sv], 0, r * 64, j * kBlockKV, bh);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    // The whole warp runs this loop and only the tcgen05 instructions are predicated on one
    // elected lane: see umma_ss_f16_if.
    if (leader && n > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(kPairQ, kBlockKV, true, false, false);  // Q K^T: both K-major
      constexpr uint32_t idesc_o = make_idesc_f16(kPairQ, kD, true, false, true);         // P V: V is MN-major
      const uint32_t el = elect_one() ? 1u : 0u;
      bool ok = true;
      auto wait = [&](uint64_t* bar, uint32_t parity, int site) {
        const bool w = mbar_wait<true>(bar, parity, status, SILE_ERR_TIMEOUT, site);
        return __all_sync(0xffffffffu, w);
      };

      // Descriptors name offsets that are valid in both CTAs' shared memory; they are built once
      // and inside the unrolled loops only a constant is added to the start-address field.
      const uint64_t q_desc = make_smem_desc_sw128(smem_u32(smem + kSmemQ), 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem + kSmemK), 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem + kSmemV), kVStageBytes, 1024);

      auto issue_s = [&](int j) -> bool {
        // S_j (256 x 128 keys) = Q (two 64-wide head-dim panels) * K_j^T, 64 keys from each CTA
        const int sk = j % kStagesK, b = j % kBufS;
        if (!wait(&k_full[sk], (j / kStagesK) & 1, 3)) return false;
        tcgen05_fence_after();
        const uint64_t db = k_desc0 + sk * (kKStageBytes >> 4);
        const uint32_t d = tmem_s[b];
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off_q = (kk >> 2) * (kQPanelBytes >> 4) + (kk & 3) * 2;  // in 16-byte units
          const uint32_t off_k = (kk >> 2) * (kKPanelBytes >> 4) + (kk & 3) * 2;
          umma_ss_f16_if<2>(el, d, q_desc + off_q, db + off_k, idesc_s, kk != 0 ? 1u : 0u);
        }
        commit_both(el, &s_full[b]);
        commit_both(el, &k_empty[sk]);
        return true;
      };

      ok = wait(q_full, 0, 4);
      for (int j = 0; j < kBufS && j < n && ok; ++j) ok = issue_s(j);
      for (int j = 0; j < n && ok; ++j) {
        const int b = j % kBufS, sv = j % kStagesV;
        if (!wait(&v_full[sv], (j / kStagesV) & 1, 5)) { ok = false; break; }
        if (!wait(&p_full[b], (j / kBufS) & 1, 6)) { ok = false; break; }
        tcgen05_fence_after();
        // O (256 x 128 d) += P_j (TMEM, 8 columns per 16 keys) * V_j (rows = keys, 2048 B per 16
        // keys), 64 head-dim columns from each CTA
        const uint64_t db = v_desc0 + sv * (kVStageBytes >> 4);
        const uint32_t a = tmem_s[b];
        umma_ts_f16_if<2>(el, tmem_o, a, db, idesc_o, j > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < kBlockKV / 16; ++kk) umma_ts_f16_if<2>(el, tmem_o, a + kk * 8, db + kk * 128, idesc_o, 1u);
        commit_both(el, &v_empty[sv]);  // also tells the softmax warps that O holds block j
        if (j + kBufS < n) ok = issue_s(j + kBufS);
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax / correction / epilogue (both CTAs, own 128 rows) ----------------
    const int quarter = warp & 3;         // TMEM lane quarter of this warp
    const int row_in_tile = quarter * 32 + lane;
    const int q_tile0 = q_base + static_cast<int>(rank) * kTileQ;
    const int q_idx = q_tile0 + row_in_tile;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t to = tmem_o + lane_off;
    float m_used = -INFINITY;  // row max (scaled, log2 domain) that P, l and O currently refer to
    float l = 0.0f;
    bool ok = true;

    for (int j = 0; j < n; ++j) {
      const int b = j % kBufS;
      const uint32_t use = (j / kBufS) & 1;  // parity of this use of buffer b
      const uint32_t ts = tmem_s[b] + lane_off;
      if (!mbar_wait<true>(&s_full[b], use, status, SILE_ERR_TIMEOUT, 7)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();

      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(ts + c * 32, sr[c]);
      tcgen05_wait_ld();

      const int kv0 = j * kBlockKV;
      const bool need_mask = (kv0 + kBlockKV > p.s) || (p.causal && kv0 + kBlockKV - 1 > q_tile0);
      if (need_mask) {
        const int limit = p.causal ? min(q_idx, p.s - 1) : p.s - 1;  // last visible key index
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kv0 + c * 32 + i > limit) sr[c][i] = 0xff800000u;  // -inf
      }

      float mx[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) mx[c] = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          mx[2 * c] = max3(mx[2 * c], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
          mx[2 * c + 1] = max3(mx[2 * c + 1], __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
        }
      }
      const float m_blk = fmaxf(max3(mx[0], mx[1], mx[2]), max3(max3(mx[3], mx[4], mx[5]), mx[6], mx[7])) * p.scale_log2;
      const float m_new = fmaxf(m_used, m_blk);
      const bool rescale = (m_new - m_used > kRescaleThreshold) || (m_used == -INFINITY);  // NaN-safe: inf - (-inf)
      float alpha = 1.0f;
      if (rescale) {
        alpha = (m_used == -INFINITY) ? 0.0f : ex2(m_used - m_new);
        m_used = m_new;
      }
      const float m_sub = (m_used == -INFINITY) ? 0.0f : m_used;

      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
        // P_{j-1} V_{j-1} (and with it every earlier one) must have landed in O before it is scaled.
        // The commit that frees V stage (j-1) % kStagesV says so; these warps only observe that
        // barrier.  It cannot be a phase ahead (P_j V_j needs the P this step has yet to write)
        // nor be mistaken for the previous phase (a wait on a parity returns only once the phase
        // of that parity has completed).
        if (!mbar_wait<true>(&v_empty[(j - 1) % kStagesV], ((j - 1) / kStagesV) & 1, status, SILE_ERR_TIMEOUT, 8)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t orow[32];
          tmem_ld_32x32b_x32(to + c * 32, orow);
          tcgen05_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
          tmem_st_32x32b_x32(to + c * 32, orow);
        }
        tcgen05_wait_st();
      }

      // P = 2^(s * scale_log2 - m), staged per 32-key chunk so that its 32 MUFU ops are independent
      // and issue back to back (FMA -> MUFU -> ADD per element leaves the warp waiting on MUFU
      // latency between elements).
      float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; ++i) sr[c][i] = __float_as_uint(fmaf(__uint_as_float(sr[c][i]), p.scale_log2, -m_sub));
#pragma unroll
        for (int i = 0; i < 32; ++i) sr[c][i] = __float_as_uint(ex2(__uint_as_float(sr[c][i])));
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float p0 = __uint_as_float(sr[c][4 * i]), p1 = __uint_as_float(sr[c][4 * i + 1]);
          const float p2 = __uint_as_float(sr[c][4 * i + 2]), p3 = __uint_as_float(sr[c][4 * i + 3]);
          sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
          pk[2 * i] = pack_bf16x2(p0, p1);
          pk[2 * i + 1] = pack_bf16x2(p2, p3);
        }
        tmem_st_32x32b_x16(ts + c * 16, pk);
      }
      sum0 += sum2;
      sum1 += sum3;
      l = l * alpha + (sum0 + sum1);
      tcgen05_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      // the leader's barrier: 4 warps from each CTA.  The waiter is in another CTA, so the arrive
      // carries a release at cluster scope (the PTX memory model gives no cross-CTA ordering to a
      // CTA-scope release); it costs ~850 cycles per arrive, which this variant can afford.
      if (lane == 0) mbar_arrive_cluster(&p_full[b], 0);
    }

    if (ok && n > 0) {
      if (!mbar_wait<true>(&v_empty[(n - 1) % kStagesV], ((n - 1) / kStagesV) & 1, status, SILE_ERR_TIMEOUT, 9)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tcgen05_fence_after();
        const float inv_l = 1.0f / l;
        __nv_bfloat16* dst = o + (static_cast<int64_t>(bh) * p.s + q_idx) * p.row_stride;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t orow[32];
          tmem_ld_32x32b_x32(to + c * 32, orow);
          tcgen05_wait_ld();
          if (q_idx < p.s) {
            uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(orow[8 * i]) * inv_l, __uint_as_float(orow[8 * i + 1]) * inv_l);
              v.y = pack_bf16x2(__uint_as_float(orow[8 * i + 2]) * inv_l, __uint_as_float(orow[8 * i + 3]) * inv_l);
              v.z = pack_bf16x2(__uint_as_float(orow[8 * i + 4]) * inv_l, __uint_as_float(orow[8 * i + 5]) * inv_l);
              v.w = pack_bf16x2(__uint_as_float(orow[8 * i + 6]) * inv_l, __uint_as_float(orow[8 * i + 7]) * inv_l);
              d4[i] = v;
            }
          }
        }
      }
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

}  // namespace

int attention_pair_launch(const AttnProblem& a, cudaStream_t stream) {
  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;

  CUtensorMap tq, tk, tv;
  const uint64_t dims[3] = {static_cast<uint64_t>(kD), static_cast<uint64_t>(a.s), static_cast<uint64_t>(a.bh)};
  const uint64_t strides[2] = {static_cast<uint64_t>(kD) * 2, static_cast<uint64_t>(a.s) * kD * 2};
  const uint32_t box_q[3] = {64, kTileQ, 1};
  const uint32_t box_k[3] = {64, kBlockKV / 2, 1};
  const uint32_t box_v[3] = {64, kBlockKV, 1};
  if (int rc = encode_tensor_map(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.q, dims, strides, box_q, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = encode_tensor_map(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.k, dims, strides, box_k, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = encode_tensor_map(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.v, dims, strides, box_v, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;

  PairParams p{};
  p.s = static_cast<int>(a.s);
  p.bh = static_cast<int>(a.bh);
  p.num_qblocks = static_cast<int>((a.s + kPairQ - 1) / kPairQ);
  p.causal = a.causal ? 1 : 0;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.row_stride = kD;

  SILE_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  const int64_t clusters = static_cast<int64_t>(p.bh) * p.num_qblocks;
  if (2 * clusters > 0x7fffffffll) return fail(SILE_ERR_INVALID, "attention: too many blocks");
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SILE_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_fwd_pair_kernel, tq, tk, tv, static_cast<__nv_bfloat16*>(a.o), p, status));
  note_kernel("attn_fwd_pair_kernel", cfg.gridDim.x, cfg.blockDim.x, cfg.dynamicSmemBytes);
  return SILE_OK;
}

}  // namespace sile
