// Fused attention forward for sm_100a, bf16 in/out, head_dim 128: the kernel of attn_sm100.cu with
// the softmax of every Q tile spread over EIGHT warps instead of four.
//
// There, thread r of a tile's four softmax warps owns row r and all 128 scores of a key block,
// and the chain S -> softmax -> P V -> next S of a tile is bounded by what one warp can issue for
// its 128 scores per row (two softmax warps per scheduler leave the issue slots 58 % empty).
// Here two warps share a row quarter: warps 2..9 take keys [0, 64) of every block ("half 0"),
// warps 10..17 keys [64, 128) ("half 1"); warp w and warp w + 8 reach the same TMEM lanes.  Per
// block the two threads of a row exchange their partial row maxima through shared memory (double
// buffered, one 64-thread named barrier), then each exponentiates, sums and stores its own 64
// keys and publishes them as one piece of P; the row sums stay partial until the epilogue, where
// they are exchanged once.  A lazy rescale of O is split by columns between the halves, with a
// second named barrier before any piece of P is published (P V of the new block accumulates into
// all 128 columns).  The epilogue is split by 64-column panel.  Everything else -- TMA producer,
// MMA issue order, TMEM layout S0 | S1 | O0 | O1, lazy rescale threshold -- is attn_sm100.cu's.
//
// Measured 10 % behind attn_sm100.cu's kernel (batch 4 x 32 heads x 4096: 1170 against 1300
// TFLOP/s), so it is opt-in (SILE_CUDA_ATTN_KERNEL=split).  With 18 warps a thread has 96
// registers, not enough for 64 scores next to the 16 packed words of P (holding them spilled 400
// bytes and ran at 600 TFLOP/s), so the scores are read from tensor memory twice: once for the
// maximum, once for the exponentials.
//
// Both threads of a row always execute the same sequence of named barriers: a bounded wait that
// gave up is reported to the partner THROUGH the exchange, and both leave the loop together.
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
constexpr int kThreads = 576;  // TMA warp, MMA warp, 2 tiles x 2 halves x 4 softmax warps
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + 2 * kTileBytes;
constexpr int kSmemV = kSmemK + kStagesKV * kTileBytes;
constexpr int kSmemBar = kSmemV + kStagesKV * kTileBytes;
constexpr int kSmemXchg = kSmemBar + 256;                 // [2 buffers][2 tiles][2 halves][128 rows] floats
constexpr int kSmemBytes = kSmemXchg + 2 * 2 * 2 * 128 * 4 + 8 * 4 + 1024;  // + one give-up flag per pair of warps
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// P_t reaches the MMA warp in two pieces, keys [0, 64) from half 0 and keys [64, 128) from half 1,
// each on its own barrier (four arrivals: the four warps of that half).
constexpr unsigned kPublishMask = 0xA;
__host__ __device__ constexpr int piece_of_chunk(int c) { return c >> 1; }

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
attn_fwd_split_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
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
    for (int i = 0; i < 8; ++i) mbar_init(&p_full[i], 4);  // one arrival per softmax warp of the tile's half
    for (int i = 0; i < 8; ++i) reinterpret_cast<int*>(smem + kSmemXchg + 4096)[i] = 0;
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
        // O_t += P_t (TMEM, 8 columns per 16 keys; keys [0, 64) at columns [0, 32) and keys [64, 128) at
        // columns [64, 96) of S_t, each half over its own scores) * V_st (rows = keys, 2048 B per 16 keys;
        // d panels 16 KiB apart), piece by piece as the softmax warps publish P_t
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
            umma_ts_f16_if<1>(el, d, a + (kk >> 2) * 64 + (kk & 3) * 8, db + kk * 128, idesc_o, (accumulate || kk != 0) ? 1u : 0u);
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
    const int half = (warp - 2) >> 3;       // keys [64 * half, 64 * half + 64) of every block
    const int t = ((warp - 2) >> 2) & 1;    // Q tile of this group of four warps
    const int quarter = warp & 3;           // TMEM lane quarter of this warp (warp w and w + 8 share it)
    const int row_in_tile = quarter * 32 + lane;
    const int q_idx = q_base + t * kTileQ + row_in_tile;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t ts = tmem_s[t] + lane_off;
    const uint32_t to = tmem_o[t] + lane_off;
    const int n = n_kv[t];
    // exchange slots of this row: [buffer][tile][half][row]; the partner's slot is the other half's
    float* xchg = reinterpret_cast<float*>(smem + kSmemXchg);
    const int slot_mine = (t * 2 + half) * 128 + row_in_tile;
    const int slot_other = (t * 2 + (half ^ 1)) * 128 + row_in_tile;
    int* pair_fail = reinterpret_cast<int*>(xchg + 1024) + t * 4 + quarter;  // set by a warp of the pair whose wait gave up
    const uint32_t pair_bar = 1 + t * 4 + quarter;  // named barrier of the two warps that share these rows
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory"); };
    float m_used = -INFINITY;  // row max (scaled, log2 domain) that P, l and O currently refer to
    float l = 0.0f;            // this half's share of the row sum
    bool ok = true;

    for (int j = 0; j < n; ++j) {
      if (!mbar_wait(&s_full[t], j & 1, status, SILE_ERR_TIMEOUT)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      float m_blk = -INFINITY;
      const int kv0 = j * kBlockKV + half * 64;
      const bool need_mask = (kv0 + 64 > p.s) || (p.causal && kv0 + 64 - 1 > q_base + t * kTileQ);
      const int limit = p.causal ? min(q_idx, p.s - 1) : p.s - 1;  // last visible key index
      if (ok) {
        tcgen05_fence_after();
        // pass 1: the maximum of this half's 64 scores, 32 at a time (they are read again below:
        // holding all 64 next to the 16 packed words of P does not fit the 96 registers that 18
        // warps leave a thread)
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t sr[32];
          tmem_ld_32x32b_x32(ts + half * 64 + c * 32, sr);
          tcgen05_wait_ld();
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kv0 + c * 32 + i > limit) sr[i] = 0xff800000u;  // -inf
          }
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            mx0 = max3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
            mx1 = max3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
            mx2 = max3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
            mx3 = max3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
          }
        }
        m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      }
      // Row maximum over both halves.  A warp whose wait gave up raises the pair's flag; both warps
      // then see it and leave together, after the same number of named barriers.
      xchg[(j & 1) * 512 + slot_mine] = m_blk;
      if (!ok && lane == 0) *reinterpret_cast<volatile int*>(pair_fail) = 1;
      pair_sync();
      const float m_other = xchg[(j & 1) * 512 + slot_other];
      ok = *reinterpret_cast<volatile int*>(pair_fail) == 0;
      if (!ok) break;
      m_blk = fmaxf(m_blk, m_other);

      const float m_new = fmaxf(m_used, m_blk);
      const bool rescale = (m_new - m_used > kRescaleThreshold) || (m_used == -INFINITY);  // NaN-safe: inf - (-inf)
      float alpha = 1.0f;
      if (rescale) {
        alpha = (m_used == -INFINITY) ? 0.0f : ex2(m_used - m_new);
        m_used = m_new;
      }
      const float m_sub = (m_used == -INFINITY) ? 0.0f : m_used;

      // The decision is the same in both warps of the pair (same rows, same maxima).
      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
        // O_t already holds block j-1: S_t of block j was issued after P_{j-1} V_{j-1}, MMAs
        // retire in issue order, and the s_full wait above ordered this thread after all of them.
        // This half rescales its 64 columns; no piece of P may be published before both halves
        // are done, because P V of block j accumulates into all 128 columns.
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t orow[32];
          tmem_ld_32x32b_x32(to + half * 64 + c * 32, orow);
          tcgen05_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
          tmem_st_32x32b_x32(to + half * 64 + c * 32, orow);
        }
        tcgen05_wait_st();
        tcgen05_fence_before();
        pair_sync();
        tcgen05_fence_after();
      }

      // pass 2: P = 2^(s * scale_log2 - m) per 32-key chunk, its 32 MUFU ops independent and issued
      // back to back.  P (bf16 pairs) goes to columns [64 * half, 64 * half + 32) of S_t, over
      // scores of this half that have just been read.
      float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sr[32];
        tmem_ld_32x32b_x32(ts + half * 64 + c * 32, sr);
        tcgen05_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kv0 + c * 32 + i > limit) sr[i] = 0xff800000u;  // -inf
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) sr[i] = __float_as_uint(fmaf(__uint_as_float(sr[i]), p.scale_log2, -m_sub));
#pragma unroll
        for (int i = 0; i < 32; ++i) sr[i] = __float_as_uint(ex2(__uint_as_float(sr[i])));
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float p0 = __uint_as_float(sr[4 * i]), p1 = __uint_as_float(sr[4 * i + 1]);
          const float p2 = __uint_as_float(sr[4 * i + 2]), p3 = __uint_as_float(sr[4 * i + 3]);
          sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
          pk[2 * i] = pack_bf16x2(p0, p1);
          pk[2 * i + 1] = pack_bf16x2(p2, p3);
        }
        // P of chunk c lands on columns [16 c, 16 c + 16) of this half: on chunk 0's scores, which
        // this pass has read by then, never on scores still to be read
        tmem_st_32x32b_x16(ts + half * 64 + c * 16, pk);
      }
      tcgen05_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t * 4 + half]);
      sum0 += sum2;
      sum1 += sum3;
      l = l * alpha + (sum0 + sum1);
    }

    if (n > 0) {
      // Row sum over both halves (buffer n & 1: the one the last block did not use); a warp whose
      // wait gave up raises the pair's flag and both leave.
      if (ok && !mbar_wait(&o_done[t], 0, status, SILE_ERR_TIMEOUT)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      xchg[(n & 1) * 512 + slot_mine] = l;
      if (!ok && lane == 0) *reinterpret_cast<volatile int*>(pair_fail) = 1;
      pair_sync();
      const float l_other = xchg[(n & 1) * 512 + slot_other];
      ok = *reinterpret_cast<volatile int*>(pair_fail) == 0;
      if (ok) {
        tcgen05_fence_after();
        // O = acc / l goes out through shared memory: this warp's 32 rows of its 64-column panel are
        // converted, written in the 128-byte swizzle into the (now idle) shared memory of its own Q
        // tile, and lane 0 issues one TMA store per destination.
        const float inv_l = 1.0f / (l + l_other);
        uint8_t* stage = smem + kSmemQ + t * kTileBytes + half * kPanelBytes + quarter * 32 * 128;
        const int row0 = q_base + t * kTileQ + quarter * 32;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t orow[32];
          tmem_ld_32x32b_x32(to + half * 64 + c * 32, orow);
          tcgen05_wait_ld();
          const uint32_t row_addr = smem_u32(stage) + lane * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t v0 = pack_bf16x2(__uint_as_float(orow[8 * i]) * inv_l, __uint_as_float(orow[8 * i + 1]) * inv_l);
            const uint32_t v1 = pack_bf16x2(__uint_as_float(orow[8 * i + 2]) * inv_l, __uint_as_float(orow[8 * i + 3]) * inv_l);
            const uint32_t v2 = pack_bf16x2(__uint_as_float(orow[8 * i + 4]) * inv_l, __uint_as_float(orow[8 * i + 5]) * inv_l);
            const uint32_t v3 = pack_bf16x2(__uint_as_float(orow[8 * i + 6]) * inv_l, __uint_as_float(orow[8 * i + 7]) * inv_l);
            const uint32_t unit = c * 4 + i;  // 16-byte unit inside the 128-byte row
            const uint32_t dst = row_addr + ((unit ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v0), "r"(v1), "r"(v2), "r"(v3) : "memory");
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row0 < p.s) {
          int d = p.first_dst;
          for (int i = 0; i < p.num_dst; ++i) {
            tma_store_3d(&out_maps.map[d], stage, half * 64, row0, p.bh_offset + bh);
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

int attention_split_launch(const AttnProblem& a, cudaStream_t stream) {
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
    SILE_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set[current_device_slot()] = true;
  }
  const int64_t grid = static_cast<int64_t>(p.bh) * p.num_qblocks;
  if (grid > 0x7fffffffll) return fail(SILE_ERR_INVALID, "attention: too many blocks");
  attn_fwd_split_kernel<<<static_cast<unsigned>(grid), kThreads, kSmemBytes, stream>>>(tq, tk, tv, out_maps, p, status);
  SILE_CUDA_TRY(cudaGetLastError());
  note_kernel("attn_fwd_split_kernel", static_cast<unsigned>(grid), kThreads, kSmemBytes);
  return SILE_OK;
}

}  // namespace sile
