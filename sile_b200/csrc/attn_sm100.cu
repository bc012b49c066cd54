// Fused attention forward O = softmax(scale * Q K^T [+ causal mask]) V for sm_100a,
// bf16 in/out, head_dim 128, f32 softmax statistics.
//
// The reference has no attention kernel; this is the fused form of the op sequence its
// DSL would compose from mma / reduce_max / exp / reduce_sum tile ops
// (crates/sile-tile-ir/src/lower.rs:509-748; general mma path
// crates/sile-tile-ir/src/passes/lowering/tile_compute/mma.rs:25-260): online softmax over
// 128-key blocks with the running row max m, row sum l and an unnormalised accumulator.
//
// One CTA = one (batch*head, 256-query block) = two 128-row Q tiles, 10 warps (ptxas gives each
// thread 168 registers, enough for a softmax thread's 128 scores with a few bytes of spill):
//   warp 0        TMA producer: Q tiles once, then K_j / V_j through 2-stage rings
//   warp 1        MMA issuer:   S_t = Q_t K_j^T (smem x smem) and O_t += P_t V_j
//                 (P_t read from TMEM, V_j MN-major from smem), f32 accumulators in TMEM.
//                 The tiles are served in a fixed order (PV0 S0' PV1 S1' ...), which keeps their
//                 softmax phases apart; one issuing warp per tile was measured ~17 % slower
//                 because the tiles then fall into step and their softmaxes collide.
//   warps 2..5    softmax of Q tile 0 (thread r owns row r = TMEM lane r; a warp reaches the TMEM
//                 lane quarter warp % 4, and any four consecutive warps cover all four)
//   warps 6..9    softmax of Q tile 1
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 columns each; P_t (bf16 pairs) overwrites the
// first 64 columns of S_t.  Per tile the chain is S -> softmax -> PV -> next S; the softmax of one
// tile runs under the MMAs of the other, and P_t reaches the MMA warp in two pieces so that most
// of P V runs under the last exponentials.  O is rescaled only when the row max has grown by more
// than 2^8 since the last rescale; the same (stale) max is used for P and l, so the result is
// unchanged.  The rescale and the final 1/l normalisation are done by the softmax warps.
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "internal.h"
#include "ptx.cuh"

namespace sile {
namespace {

using namespace ptx;

constexpr int kD = 128;            // head dim
constexpr int kTileQ = 128;        // rows per Q tile (= TMEM lanes)
constexpr int kBlockQ = 2 * kTileQ;
constexpr int kBlockKV = 128;
constexpr int kPanelBytes = 128 * 64 * 2;   // one [128 rows x 64 cols] 128B-swizzled panel
constexpr int kTileBytes = 2 * kPanelBytes;  // [128 x 128] bf16
constexpr int kStagesKV = 2;
constexpr int kThreads = 320;
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + 2 * kTileBytes;
constexpr int kSmemV = kSmemK + kStagesKV * kTileBytes;
constexpr int kSmemBar = kSmemV + kStagesKV * kTileBytes;
constexpr int kSmemBytes = kSmemBar + 256 + 1024;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// P_t is handed to the MMA warp in pieces, each on its own barrier, so the first P V MMAs of a
// block run while the softmax warps still compute the later exponentials (the chain S -> softmax
// -> PV -> next S of a tile is what bounds the kernel).  P is produced in four 32-key chunks; bit c
// of kPublishMask says that a piece ends after chunk c (bit 3 is always set).  Measured on
// batch 4 x 32 heads x 4096: one piece 1222 TFLOP/s, two halves 1260, four quarters 1261,
// three quarters + one quarter 1284.
constexpr unsigned kPublishMask = 0xC;  // keys [0, 96) and [96, 128): every further signal costs a tcgen05.wait::st
static_assert((kPublishMask & 8u) != 0 && kPublishMask < 16u, "the last chunk always ends a piece");
// barrier (piece) index that chunk c belongs to
__host__ __device__ constexpr int piece_of_chunk(int c) {
  int n = 0;
  for (int i = 0; i < c; ++i) n += (kPublishMask >> i) & 1u;
  return n;
}

struct AttnParams {
  int s;          // sequence length
  int bh;         // batch * heads computed by this launch
  int num_qblocks;
  int causal;
  float scale_log2;  // scale * log2(e)
  int bh_offset;     // first head of this launch inside the destination buffers
  int num_dst;       // destination buffers (1 = local only)
  int first_dst;     // destination served first, then round-robin
};
// One tensor map per destination buffer of O ([bh_total, S, D] bf16, box 64 d x 32 rows, 128-byte
// swizzle): the local O, or with the all-gather folded in, every rank's O.
struct AttnOutMaps {
  CUtensorMap map[8];
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

// Number of 128-key blocks Q tile `t` of this CTA attends to (0 = tile is past the end).
__device__ __forceinline__ int kv_blocks_for_tile(const AttnParams& p, int q0) {
  if (q0 >= p.s) return 0;
  const int all = (p.s + kBlockKV - 1) / kBlockKV;
  if (!p.causal) return all;
  const int last_q = min(q0 + kTileQ, p.s) - 1;
  return min(all, last_q / kBlockKV + 1);
}

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ AttnOutMaps out_maps, const AttnParams p,
                int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemBar);
  uint64_t* q_full = bars;           // [2]
  uint64_t* k_full = bars + 2;       // [2]
  uint64_t* k_empty = bars + 4;      // [2]
  uint64_t* v_full = bars + 6;       // [2]
  uint64_t* v_empty = bars + 8;      // [2]
  uint64_t* s_full = bars + 10;      // [2] S_t written by the tensor core
  uint64_t* p_full = bars + 12;      // [2][4] piece c of P_t written (and O_t rescaled) by the softmax warps
  uint64_t* o_done = bars + 20;      // [2] O_t += P_t V_j finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  // Block order: heads are taken in groups of kHeadGroup; inside a group the late query blocks
  // (heavy under a causal mask) of every head come first.  Concurrently resident CTAs then share
  // the K/V of a few heads in L2, and the blocks that finish last are the light ones.
  constexpr int kHeadGroup = 8;
  const int group = blockIdx.x / (kHeadGroup * p.num_qblocks);
  const int in_group = blockIdx.x - group * kHeadGroup * p.num_qblocks;
  const int heads_here = min(kHeadGroup, p.bh - group * kHeadGroup);
  const int bh = group * kHeadGroup + in_group % heads_here;
  const int qblk = p.num_qblocks - 1 - in_group / heads_here;
  const int q_base = qblk * kBlockQ;
  const int n_kv[2] = {kv_blocks_for_tile(p, q_base), kv_blocks_for_tile(p, q_base + kTileQ)};
  const int n_max = max(n_kv[0], n_kv[1]);

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tma_q);
    prefetch_tensormap(&tma_k);
    prefetch_tensormap(&tma_v);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&o_done[i], 1);
    }
    for (int i = 0; i < 8; ++i) mbar_init(&p_full[i], 4);  // one arrival per softmax warp of the tile
    fence_barrier_init();
    fence_proxy_async_smem();
    // The first loads go out before the CTA-wide sync (this thread initialised the barriers they
    // complete on), so they travel while tensor memory is being allocated.
    auto load_first = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int row0) {
      mbar_expect_tx(bar, kTileBytes);
      tma_load_3d(dst, map, bar, 0, row0, bh);
      tma_load_3d(dst + kPanelBytes, map, bar, 64, row0, bh);
    };
    if (n_kv[0] > 0) load_first(&tma_q, smem + kSmemQ, &q_full[0], q_base);
    if (n_max > 0) load_first(&tma_k, smem + kSmemK, &k_full[0], 0);
    if (n_kv[1] > 0) load_first(&tma_q, smem + kSmemQ + kTileBytes, &q_full[1], q_base + kTileQ);
    if (n_max > 0) load_first(&tma_v, smem + kSmemV, &v_full[0], 0);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, kTmemCols);
    tmem_relinquish<1>();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_o[2] = {tmem_base + 256, tmem_base + 384};

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      bool ok = true;
      auto load_tile = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int row0) {
        mbar_expect_tx(bar, kTileBytes);
        tma_load_3d(dst, map, bar, 0, row0, bh);
        tma_load_3d(dst + kPanelBytes, map, bar, 64, row0, bh);
      };
      // Q tiles and block 0 of K / V were requested before the CTA-wide sync above.
      for (int j = 1; j < n_max && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1u, status, SILE_ERR_TIMEOUT)) { ok = false; break; }
        load_tile(&tma_k, smem + kSmemK + st * kTileBytes, &k_full[st], j * kBlockKV);
        if (!mbar_wait(&v_empty[st], ph ^ 1u, status, SILE_ERR_TIMEOUT)) { ok = false; break; }
        load_tile(&tma_v, smem + kSmemV + st * kTileBytes, &v_full[st], j * kBlockKV);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp runs this loop (waits included) and only the tcgen05 instructions are
    // predicated on one elected lane: see umma_ss_f16_if.
    if (n_max > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(kTileQ, kBlockKV, true, false, false);  // Q K^T: both K-major
      constexpr uint32_t idesc_o = make_idesc_f16(kTileQ, kD, true, false, true);         // P V: V is MN-major
      const uint32_t q_addr = smem_u32(smem + kSmemQ);
      const uint32_t k_addr = smem_u32(smem + kSmemK);
      const uint32_t v_addr = smem_u32(smem + kSmemV);
      const uint32_t el = elect_one() ? 1u : 0u;
      bool ok = true;

      // Descriptors are built once; inside the unrolled loops only a constant is added to the
      // 14-bit start-address field (a 128 x 128 x 16 MMA runs for 64 cycles: an issue sequence
      // slower than that starves the tensor pipe).
      const uint64_t q_desc[2] = {make_smem_desc_sw128(q_addr, 16, 1024), make_smem_desc_sw128(q_addr + kTileBytes, 16, 1024)};
      const uint64_t k_desc[2] = {make_smem_desc_sw128(k_addr, 16, 1024), make_smem_desc_sw128(k_addr + kTileBytes, 16, 1024)};
      const uint64_t v_desc[2] = {make_smem_desc_sw128(v_addr, kPanelBytes, 1024),
                                  make_smem_desc_sw128(v_addr + kTileBytes, kPanelBytes, 1024)};
      auto wait = [&](uint64_t* bar, uint32_t parity) {
        const bool w = mbar_wait(bar, parity, status, SILE_ERR_TIMEOUT);
        return __all_sync(0xffffffffu, w);
      };
      auto issue_s = [&](int t, int st) {
        // S_t = Q_t (128 x 128, two 64-wide k panels) * K_st^T
        const uint64_t da = q_desc[t], db = k_desc[st];
        const uint32_t d = tmem_s[t];
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          constexpr int kPanelUnits = kPanelBytes >> 4;
          const uint32_t off = (kk >> 2) * kPanelUnits + (kk & 3) * 2;  // in 16-byte units
          umma_ss_f16_if<1>(el, d, da + off, db + off, idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit_if<1>(el, smem_u32(&s_full[t]));
      };
      auto issue_pv = [&](int t, int st, uint32_t parity, bool accumulate, bool last) {
        // O_t += P_t (TMEM, 8 columns per 16 keys) * V_st (rows = keys, 2048 B per 16 keys; d panels 16 KiB apart),
        // piece by piece as the softmax warps publish P_t
        const uint64_t db = v_desc[st];
        const uint32_t d = tmem_o[t], a = tmem_s[t];
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // 32-key chunks of P, two MMAs each
          if (c == 0 || ((kPublishMask >> (c - 1)) & 1u)) {
            if (!wait(&p_full[t * 4 + piece_of_chunk(c)], parity)) return false;
            tcgen05_fence_after();
          }
#pragma unroll
          for (int kk = 2 * c; kk < 2 * c + 2; ++kk)
            umma_ts_f16_if<1>(el, d, a + kk * 8, db + kk * 128, idesc_o, (accumulate || kk != 0) ? 1u : 0u);
        }
        if (last) umma_commit_if<1>(el, smem_u32(&o_done[t]));  // only the epilogue waits for O; see the rescale comment below
        return true;
      };

      // prologue: S_0 for both tiles
      if (n_kv[0] > 0) ok = ok && wait(&q_full[0], 0);
      ok = ok && wait(&k_full[0], 0);
      if (ok) {
        tcgen05_fence_after();
        if (n_kv[0] > 0) issue_s(0, 0);
        if (n_kv[1] > 0) {
          ok = wait(&q_full[1], 0);
          if (ok) {
            tcgen05_fence_after();
            issue_s(1, 0);
          }
        }
        umma_commit_if<1>(el, smem_u32(&k_empty[0]));
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int st_n = (j + 1) & 1;
        const uint32_t ph_n = ((j + 1) >> 1) & 1;
        if (!wait(&v_full[st], ph)) { ok = false; break; }
        if (j < n_kv[0]) {
          if (!issue_pv(0, st, j & 1, j > 0, j + 1 == n_kv[0])) { ok = false; break; }
        }
        if (j + 1 < n_max) {
          if (!wait(&k_full[st_n], ph_n)) { ok = false; break; }
          tcgen05_fence_after();
        }
        if (j + 1 < n_kv[0]) issue_s(0, st_n);
        if (j < n_kv[1]) {
          if (!issue_pv(1, st, j & 1, j > 0, j + 1 == n_kv[1])) { ok = false; break; }
        }
        umma_commit_if<1>(el, smem_u32(&v_empty[st]));
        if (j + 1 < n_kv[1]) issue_s(1, st_n);
        if (j + 1 < n_max) umma_commit_if<1>(el, smem_u32(&k_empty[st_n]));
      }
    }
    __syncwarp();
  } else if (warp >= 2) {
    // ---------------- softmax / correction / epilogue ----------------
    const int t = (warp - 2) >> 2;        // Q tile of this group of four warps
    const int quarter = warp & 3;         // TMEM lane quarter of this warp
    const int row_in_tile = quarter * 32 + lane;
    const int q_idx = q_base + t * kTileQ + row_in_tile;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t ts = tmem_s[t] + lane_off;
    const uint32_t to = tmem_o[t] + lane_off;
    const int n = n_kv[t];
    float m_used = -INFINITY;  // row max (scaled, log2 domain) that P, l and O currently refer to
    float l = 0.0f;
    bool ok = true;

    for (int j = 0; j < n; ++j) {
      if (!mbar_wait(&s_full[t], j & 1, status, SILE_ERR_TIMEOUT)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();

      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(ts + c * 32, sr[c]);
      tcgen05_wait_ld();

      const int kv0 = j * kBlockKV;
      const bool need_mask = (kv0 + kBlockKV > p.s) || (p.causal && kv0 + kBlockKV - 1 > q_base + t * kTileQ);
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
      // latency between elements).  A chunk that ends a piece is published as soon as its store to
      // tensor memory has landed.
      float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
      auto publish = [&](int c) {
        tcgen05_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t * 4 + piece_of_chunk(c)]);
      };
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
        if ((kPublishMask >> c) & 1u) publish(c);
      }
      sum0 += sum2;
      sum1 += sum3;
      l = l * alpha + (sum0 + sum1);
    }

    if (ok && n > 0) {
      if (!mbar_wait(&o_done[t], 0, status, SILE_ERR_TIMEOUT)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tcgen05_fence_after();
        // O = acc / l goes out through shared memory: this warp's 32 rows are converted, written in
        // the 128-byte swizzle into the (now idle) shared memory of its own Q tile, and lane 0 issues
        // one TMA store per 64-wide head-dim panel and destination.  Global (and NVLink) writes are
        // full 128-byte lines, rows past the end of the sequence are clipped by the tensor map, and
        // with several destinations this is the all-gather of O.
        const float inv_l = 1.0f / l;
        uint8_t* stage = smem + kSmemQ + t * kTileBytes + quarter * 32 * 128;  // + panel * kPanelBytes
        const int row0 = q_base + t * kTileQ + quarter * 32;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t orow[32];
          tmem_ld_32x32b_x32(to + c * 32, orow);
          tcgen05_wait_ld();
          const uint32_t row_addr = smem_u32(stage + (c >> 1) * kPanelBytes) + lane * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t v0 = pack_bf16x2(__uint_as_float(orow[8 * i]) * inv_l, __uint_as_float(orow[8 * i + 1]) * inv_l);
            const uint32_t v1 = pack_bf16x2(__uint_as_float(orow[8 * i + 2]) * inv_l, __uint_as_float(orow[8 * i + 3]) * inv_l);
            const uint32_t v2 = pack_bf16x2(__uint_as_float(orow[8 * i + 4]) * inv_l, __uint_as_float(orow[8 * i + 5]) * inv_l);
            const uint32_t v3 = pack_bf16x2(__uint_as_float(orow[8 * i + 6]) * inv_l, __uint_as_float(orow[8 * i + 7]) * inv_l);
            const uint32_t unit = (c & 1) * 4 + i;  // 16-byte unit inside the 128-byte row
            const uint32_t dst = row_addr + ((unit ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v0), "r"(v1), "r"(v2), "r"(v3) : "memory");
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row0 < p.s) {
          int d = p.first_dst;
          for (int i = 0; i < p.num_dst; ++i) {
            tma_store_3d(&out_maps.map[d], stage, 0, row0, p.bh_offset + bh);
            tma_store_3d(&out_maps.map[d], stage + kPanelBytes, 64, row0, p.bh_offset + bh);
            if (++d == p.num_dst) d = 0;
          }
          tma_store_commit();
          tma_store_wait_all<0>();
        }
        __syncwarp();
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    if (*reinterpret_cast<volatile int*>(status) != 0) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {
      }
    }
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

}  // namespace

int attention_launch(const AttnProblem& a, cudaStream_t stream) {
  if (!a.q || !a.k || !a.v || (!a.o && a.num_peers == 0)) return fail(SILE_ERR_INVALID, "attention: null buffer");
  if (a.num_peers < 0 || a.num_peers > 8) return fail(SILE_ERR_INVALID, "attention: at most 8 destinations");
  if (a.bh <= 0 || a.s <= 0) return fail(SILE_ERR_INVALID, "attention: non-positive dimension");
  if (a.d != kD) return fail(SILE_ERR_UNSUPPORTED, "attention: head_dim %lld not supported (128 only)", (long long)a.d);
  if (a.s > (1 << 24) || a.bh > (1 << 24)) return fail(SILE_ERR_INVALID, "attention: dimension too large");
  for (const void* ptr : {a.q, a.k, a.v, static_cast<const void*>(a.o)})
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return fail(SILE_ERR_UNSUPPORTED, "attention: buffers must be 16-byte aligned");
  for (int i = 0; i < a.num_peers; ++i)
    if (!a.peer_o[i] || reinterpret_cast<uintptr_t>(a.peer_o[i]) % 16 != 0)
      return fail(SILE_ERR_INVALID, "attention: destination %d is null or not 16-byte aligned", i);
  if (a.num_peers > 0 && (a.bh_offset < 0 || a.bh_offset + a.bh > a.bh_total))
    return fail(SILE_ERR_INVALID, "attention: heads [%lld, %lld) do not fit %lld", (long long)a.bh_offset, (long long)(a.bh_offset + a.bh), (long long)a.bh_total);
  if (!(a.scale > 0.0f)) return fail(SILE_ERR_INVALID, "attention: scale must be positive");

  // Kernel choice.  The default is this file's kernel, one CTA per (head, 256-query block).
  // SILE_CUDA_ATTN_KERNEL=persistent selects the persistent kernel (attn_persist_sm100.cu: one
  // CTA per SM walking a queue of items, the next item's first Q K^T issued under the current
  // item's epilogue; measured 2-4 % behind on 4096- and 8192-long sequences, level at 1024),
  // =pair the CTA-pair kernel (attn_pair_sm100.cu: one Q tile per SM, K / V shared by the pair,
  // three S buffers; its single softmax warp per scheduler is latency-bound, ~18 % behind),
  // =split the kernel with eight softmax warps per tile (attn_split_sm100.cu, ~10 % behind).
  // Read on every launch.
  const char* which = std::getenv("SILE_CUDA_ATTN_KERNEL");
  if (which && std::strcmp(which, "pair") == 0 && a.num_peers == 0) return attention_pair_launch(a, stream);
  if (which && std::strcmp(which, "persistent") == 0) return attention_persistent_launch(a, stream);
  if (which && std::strcmp(which, "split") == 0) return attention_split_launch(a, stream);

  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;

  CUtensorMap tq, tk, tv;
  const uint64_t dims[3] = {static_cast<uint64_t>(kD), static_cast<uint64_t>(a.s), static_cast<uint64_t>(a.bh)};
  const uint64_t strides[2] = {static_cast<uint64_t>(kD) * 2, static_cast<uint64_t>(a.s) * kD * 2};
  const uint32_t box[3] = {64, 128, 1};
  if (int rc = encode_tensor_map(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = encode_tensor_map(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.k, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = encode_tensor_map(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.v, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;

  AttnParams p{};
  p.s = static_cast<int>(a.s);
  p.bh = static_cast<int>(a.bh);
  p.num_qblocks = static_cast<int>((a.s + kBlockQ - 1) / kBlockQ);
  p.causal = a.causal ? 1 : 0;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.bh_offset = static_cast<int>(a.num_peers > 0 ? a.bh_offset : 0);
  p.num_dst = a.num_peers > 0 ? a.num_peers : 1;
  p.first_dst = a.num_peers > 0 ? a.peer_first : 0;

  AttnOutMaps out_maps;
  {
    const uint64_t bh_total = static_cast<uint64_t>(a.num_peers > 0 ? a.bh_total : a.bh);
    const uint64_t odims[3] = {static_cast<uint64_t>(kD), static_cast<uint64_t>(a.s), bh_total};
    const uint32_t obox[3] = {64, 32, 1};
    for (int i = 0; i < p.num_dst; ++i) {
      void* base = a.num_peers > 0 ? a.peer_o[i] : a.o;
      if (int rc = encode_tensor_map(&out_maps.map[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, odims, strides, obox, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    }
    for (int i = p.num_dst; i < 8; ++i) out_maps.map[i] = out_maps.map[0];
  }

  static bool attr_set[kMaxDevices] = {};
  if (!attr_set[current_device_slot()]) {
    SILE_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set[current_device_slot()] = true;
  }
  const int64_t grid = static_cast<int64_t>(p.bh) * p.num_qblocks;
  if (grid > 0x7fffffffll) return fail(SILE_ERR_INVALID, "attention: too many blocks");
  attn_fwd_kernel<<<static_cast<unsigned>(grid), kThreads, kSmemBytes, stream>>>(tq, tk, tv, out_maps, p, status);
  SILE_CUDA_TRY(cudaGetLastError());
  note_kernel("attn_fwd_kernel", static_cast<unsigned>(grid), kThreads, kSmemBytes);
  return SILE_OK;
}

}  // namespace sile
