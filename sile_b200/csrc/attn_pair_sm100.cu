// Fused attention forward for sm_100a, CTA-pair form: two CTAs of a cluster (two SMs) work on
// 512 consecutive query rows of one (batch, head) and SHARE every K / V block.
//
// Same algorithm and numerics as the single-CTA kernel in attn_sm100.cu (online softmax over
// 128-key blocks, f32 statistics, lazily rescaled accumulator).  What changes is who holds what:
//   * each CTA owns two 128-row Q tiles (rows [256 t + 128 r, +128) of the 512, t = tile,
//     r = CTA rank), their S / P / O in its own tensor memory, and the softmax of those rows;
//   * of every K block each CTA stages only its 64 keys, of every V block only its 64 of the 128
//     head-dim columns (16 KiB per block and operand instead of 32 KiB);
//   * the MMAs are tcgen05 cta_group::2 instructions issued by the leader CTA: S_t (256 x 128) =
//     [Q_t of CTA0; Q_t of CTA1] K^T takes the N = 128 keys half from each CTA's shared memory,
//     and O_t += P_t V takes the N = 128 head-dim columns half from each.
// The pair therefore pulls each K / V byte from L2 once per 512 query rows instead of once per
// 256: with one CTA per SM the K / V stream (64 KiB per 128 keys per SM) is what the single-CTA
// kernel waits for; here it is halved and the freed shared memory doubles the ring depth (4 K and
// 4 V stages), which hides the L2 latency that two stages exposed.
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
constexpr int kTileQ = 128;         // rows per Q tile (= TMEM lanes)
constexpr int kPairQ = 2 * kTileQ;  // rows one cta_group::2 MMA covers (one tile from each CTA)
constexpr int kClusterQ = 2 * kPairQ;
constexpr int kBlockKV = 128;
constexpr int kQPanelBytes = kTileQ * 64 * 2;       // [128 rows x 64 d], 128B-swizzled
constexpr int kQTileBytes = 2 * kQPanelBytes;       // [128 x 128]
constexpr int kKPanelBytes = (kBlockKV / 2) * 64 * 2;  // this CTA's [64 keys x 64 d]
constexpr int kKStageBytes = 2 * kKPanelBytes;         // [64 keys x 128 d]
constexpr int kVStageBytes = kBlockKV * 64 * 2;        // this CTA's [128 keys x 64 d]
constexpr int kStagesK = 4;
constexpr int kStagesV = 4;
constexpr int kThreads = 384;
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + 2 * kQTileBytes;
constexpr int kSmemV = kSmemK + kStagesK * kKStageBytes;
constexpr int kSmemBar = kSmemV + kStagesV * kVStageBytes;
constexpr int kSmemBytes = kSmemBar + 512 + 1024;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct PairParams {
  int s;            // sequence length
  int bh;           // batch * heads
  int num_qblocks;  // 512-row query blocks per head
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

// Number of 128-key blocks the 256 query rows starting at q0 attend to (0 = past the end).
// Both CTAs of the pair run the same count: their MMAs are one instruction.
__device__ __forceinline__ int kv_blocks_for_rows(const PairParams& p, int q0) {
  if (q0 >= p.s) return 0;
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
  uint64_t* q_full = bars;                  // [2]
  uint64_t* k_full = q_full + 2;            // [kStagesK]
  uint64_t* k_empty = k_full + kStagesK;    // [kStagesK]
  uint64_t* v_full = k_empty + kStagesK;    // [kStagesV]
  uint64_t* v_empty = v_full + kStagesV;    // [kStagesV]
  uint64_t* s_full = v_empty + kStagesV;    // [2] S_t written by the tensor core
  uint64_t* p_full = s_full + 2;            // [2] P_t written (and O_t rescaled) by the softmax warps of both CTAs
  uint64_t* o_done = p_full + 2;            // [2] O_t += P_t V_j finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);

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
  const int q_base = qblk * kClusterQ;
  const int n_kv[2] = {kv_blocks_for_rows(p, q_base), kv_blocks_for_rows(p, q_base + kPairQ)};
  const int n_max = max(n_kv[0], n_kv[1]);

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tma_q);
    prefetch_tensormap(&tma_k);
    prefetch_tensormap(&tma_v);
    for (int i = 0; i < kStagesK; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < kStagesV; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 8);  // 4 softmax warps of tile i in each of the two CTAs
      mbar_init(&o_done[i], 1);
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
  const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_o[2] = {tmem_base + 256, tmem_base + 384};

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs; completions land on the leader's barriers) ----------------
    if (lane == 0) {
      bool ok = true;
      const int r = static_cast<int>(rank);
      auto load_q = [&](int t) {
        if (leader) mbar_expect_tx(&q_full[t], 2 * kQTileBytes);
        uint8_t* dst = smem + kSmemQ + t * kQTileBytes;
        const int row0 = q_base + t * kPairQ + r * kTileQ;
        tma_load_3d_pair(dst, &tma_q, &q_full[t], 0, 0, row0, bh);
        tma_load_3d_pair(dst + kQPanelBytes, &tma_q, &q_full[t], 0, 64, row0, bh);
      };
      auto load_k = [&](int j) {  // this CTA's 64 keys of block j, both head-dim panels
        const int st = j % kStagesK;
        if (leader) mbar_expect_tx(&k_full[st], 2 * kKStageBytes);
        uint8_t* dst = smem + kSmemK + st * kKStageBytes;
        const int row0 = j * kBlockKV + r * (kBlockKV / 2);
        tma_load_3d_pair(dst, &tma_k, &k_full[st], 0, 0, row0, bh);
        tma_load_3d_pair(dst + kKPanelBytes, &tma_k, &k_full[st], 0, 64, row0, bh);
      };
      auto load_v = [&](int j) {  // all 128 keys of block j, this CTA's 64 head-dim columns
        const int st = j % kStagesV;
        if (leader) mbar_expect_tx(&v_full[st], 2 * kVStageBytes);
        tma_load_3d_pair(smem + kSmemV + st * kVStageBytes, &tma_v, &v_full[st], 0, r * 64, j * kBlockKV, bh);
      };
      if (n_kv[0] > 0) load_q(0);
      if (n_max > 0) load_k(0);
      if (n_kv[1] > 0) load_q(1);
      if (n_max > 0) load_v(0);
      for (int j = 1; j < n_max && ok; ++j) {
        if (!mbar_wait<true>(&k_empty[j % kStagesK], ((j / kStagesK) & 1) ^ 1u, status, SILE_ERR_TIMEOUT, 1)) { ok = false; break; }
        load_k(j);
        if (!mbar_wait<true>(&v_empty[j % kStagesV], ((j / kStagesV) & 1) ^ 1u, status, SILE_ERR_TIMEOUT, 2)) { ok = false; break; }
        load_v(j);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    // The whole warp runs this loop and only the tcgen05 instructions are predicated on one
    // elected lane: see umma_ss_f16_if.
    if (leader && n_max > 0) {
      const uint32_t el = elect_one() ? 1u : 0u;
      auto wait = [&](uint64_t* bar, uint32_t parity, int site) {
        const bool w = mbar_wait<true>(bar, parity, status, SILE_ERR_TIMEOUT, site);
        return __all_sync(0xffffffffu, w);
      };
      constexpr uint32_t idesc_s = make_idesc_f16(kPairQ, kBlockKV, true, false, false);  // Q K^T: both K-major
      constexpr uint32_t idesc_o = make_idesc_f16(kPairQ, kD, true, false, true);         // P V: V is MN-major
      bool ok = true;

      // Descriptors name offsets that are valid in both CTAs' shared memory; they are built once
      // and inside the unrolled loops only a constant is added to the start-address field.
      const uint64_t q_desc[2] = {make_smem_desc_sw128(smem_u32(smem + kSmemQ), 16, 1024),
                                  make_smem_desc_sw128(smem_u32(smem + kSmemQ + kQTileBytes), 16, 1024)};
      const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem + kSmemK), 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem + kSmemV), kVStageBytes, 1024);

      auto issue_s = [&](int t, int j) {
        // S_t (256 x 128 keys) = Q_t (two 64-wide head-dim panels) * K_j^T, 64 keys from each CTA
        const uint64_t da = q_desc[t], db = k_desc0 + (j % kStagesK) * (kKStageBytes >> 4);
        const uint32_t d = tmem_s[t];
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off_q = (kk >> 2) * (kQPanelBytes >> 4) + (kk & 3) * 2;  // in 16-byte units
          const uint32_t off_k = (kk >> 2) * (kKPanelBytes >> 4) + (kk & 3) * 2;
          umma_ss_f16_if<2>(el, d, da + off_q, db + off_k, idesc_s, kk != 0 ? 1u : 0u);
        }
        commit_both(el, &s_full[t]);
      };
      auto issue_pv = [&](int t, int j, bool accumulate, bool last) {
        // O_t (256 x 128 d) += P_t (TMEM, 8 columns per 16 keys) * V_j (rows = keys, 2048 B per
        // 16 keys), 64 head-dim columns from each CTA
        const uint64_t db = v_desc0 + (j % kStagesV) * (kVStageBytes >> 4);
        const uint32_t d = tmem_o[t], a = tmem_s[t];
        umma_ts_f16_if<2>(el, d, a, db, idesc_o, accumulate ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < kBlockKV / 16; ++kk) umma_ts_f16_if<2>(el, d, a + kk * 8, db + kk * 128, idesc_o, 1u);
        if (last) commit_both(el, &o_done[t]);  // only the epilogue waits for O; see the rescale comment below
      };

      // prologue: S_0 for both tiles
      if (n_kv[0] > 0) ok = ok && wait(&q_full[0], 0, 3);
      ok = ok && wait(&k_full[0], 0, 4);
      if (ok) {
        tcgen05_fence_after();
        if (n_kv[0] > 0) issue_s(0, 0);
        if (n_kv[1] > 0) {
          ok = wait(&q_full[1], 0, 3);
          if (ok) {
            tcgen05_fence_after();
            issue_s(1, 0);
          }
        }
        commit_both(el, &k_empty[0]);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        if (!wait(&v_full[j % kStagesV], (j / kStagesV) & 1, 5)) { ok = false; break; }
        if (j < n_kv[0]) {
          if (!wait(&p_full[0], j & 1, 6)) { ok = false; break; }
          tcgen05_fence_after();
          issue_pv(0, j, j > 0, j + 1 == n_kv[0]);
        }
        if (j + 1 < n_max) {
          if (!wait(&k_full[(j + 1) % kStagesK], ((j + 1) / kStagesK) & 1, 4)) { ok = false; break; }
          tcgen05_fence_after();
        }
        if (j + 1 < n_kv[0]) issue_s(0, j + 1);
        if (j < n_kv[1]) {
          if (!wait(&p_full[1], j & 1, 6)) { ok = false; break; }
          tcgen05_fence_after();
          issue_pv(1, j, j > 0, j + 1 == n_kv[1]);
        }
        commit_both(el, &v_empty[j % kStagesV]);
        if (j + 1 < n_kv[1]) issue_s(1, j + 1);
        if (j + 1 < n_max) commit_both(el, &k_empty[(j + 1) % kStagesK]);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ---------------- softmax / correction / epilogue (both CTAs, own rows) ----------------
    const int t = (warp - 4) >> 2;        // Q tile of this warpgroup
    const int quarter = warp & 3;         // TMEM lane quarter of this warp
    const int row_in_tile = quarter * 32 + lane;
    const int q_tile0 = q_base + t * kPairQ + static_cast<int>(rank) * kTileQ;
    const int q_idx = q_tile0 + row_in_tile;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t ts = tmem_s[t] + lane_off;
    const uint32_t to = tmem_o[t] + lane_off;
    const int n = n_kv[t];
    float m_used = -INFINITY;  // row max (scaled, log2 domain) that P, l and O currently refer to
    float l = 0.0f;
    bool ok = true;

    for (int j = 0; j < n; ++j) {
      if (!mbar_wait<true>(&s_full[t], j & 1, status, SILE_ERR_TIMEOUT, 7)) ok = false;
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
        // O_t already holds block j-1: S_t of block j was issued after P_{j-1} V_{j-1}, MMAs
        // retire in issue order, and the s_full wait above ordered this thread after all of them.
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
      if (lane == 0) mbar_arrive_cluster(&p_full[t], 0);  // the leader's barrier: 4 warps from each CTA
    }

    if (ok && n > 0) {
      if (!mbar_wait<true>(&o_done[t], 0, status, SILE_ERR_TIMEOUT, 9)) ok = false;
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
  p.num_qblocks = static_cast<int>((a.s + kClusterQ - 1) / kClusterQ);
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
  return SILE_OK;
}

}  // namespace sile
