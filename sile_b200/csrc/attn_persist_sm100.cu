// Fused attention forward for sm_100a, persistent form: one CTA per SM walks a queue of
// (batch*head, 256-query block) work items, so the launch, tensor-memory allocation, first loads
// and pipeline ramp are paid once per SM instead of once per item, and the first Q K^T of a tile's
// next item runs under the epilogue of its current one.
//
// Same algorithm, numerics and inner loops as attn_fwd_kernel in attn_sm100.cu (online softmax
// over 128-key blocks, f32 statistics, P fed to the tensor core from tensor memory, lazily
// rescaled accumulator); the reference has no attention kernel, this is the fused form of the op
// sequence its DSL would compose (crates/sile-tile-ir/src/lower.rs:509-748, general mma path
// crates/sile-tile-ir/src/passes/lowering/tile_compute/mma.rs:25-260).
//
// 12 warps in three warpgroups; registers move from the first to the other two with setmaxnreg:
//   warp 0        TMA producer and scheduler: takes items from a global counter (heaviest first
//                 under a causal mask), publishes them through a 4-slot ring in shared memory,
//                 loads Q tiles per item and K_j / V_j through 2-stage rings that run on across items
//   warp 1        MMA issuer (whole warp, predicated tcgen05): S_t = Q_t K_j^T, O_t += P_t V_j
//   warps 2, 3    idle (a warpgroup is four warps)
//   warps 4..7    softmax and epilogue of Q tile 0 (thread r owns row r = TMEM lane r)
//   warps 8..11   softmax and epilogue of Q tile 1
// TMEM (512 columns): S0 | S1 | O0 | O1; P_t overwrites the first 64 columns of S_t.
//
// Item boundary: the first Q K^T of a tile's NEXT item is issued in the slot where the tile's
// next in-item Q K^T would go, right after the tile's last P V (the Q tile was reloaded as soon as
// the item's last Q K^T had read it), so it runs while the tile's softmax warps write O out:
// O * (1 / l) -> bf16 -> a 128-byte-swizzled staging buffer of the warp's own -> TMA store (one
// per destination).  The next item's first P V cannot overtake that: it waits for P, which the
// same warps produce only after they have read O.
//
// Two things measured on the way here shaped this file.  A separate correction warpgroup for the
// epilogue (and a scheduler warp) cost more than it saved: warps that mostly wait still poll, and
// on the schedulers they share with the softmax warps that was worth 5 %.  And the instruction
// cache matters: with four roles' loops unrolled the kernel ran at a 96 % instruction-cache hit
// rate against 99.4 % and every barrier hand-off took hundreds of cycles longer, so cold paths
// (the scheduler, item decoding, the epilogue) are kept out of the unrolled hot loops.
#include <cuda_bf16.h>

#include <algorithm>

#include "internal.h"
#include "ptx.cuh"

namespace sile {
namespace {

using namespace ptx;

constexpr int kD = 128;
constexpr int kTileQ = 128;
constexpr int kBlockQ = 2 * kTileQ;
constexpr int kBlockKV = 128;
constexpr int kPanelBytes = 128 * 64 * 2;
constexpr int kTileBytes = 2 * kPanelBytes;
constexpr int kThreads = 384;
constexpr int kRing = 4;  // scheduler ring slots
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + 2 * kTileBytes;
constexpr int kSmemV = kSmemK + 2 * kTileBytes;
constexpr int kSmemStage = kSmemV + 2 * kTileBytes;  // 8 softmax warps x [32 rows][128 B]: one 64-wide panel each
constexpr int kSmemBar = kSmemStage + 8 * 4096;
constexpr int kSmemBytes = kSmemBar + 512 + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// registers per thread after the warpgroups have traded: 128 * 104 + 256 * 200 = 64512 of the
// 64512 the kernel is launched with (384 threads x 168)
constexpr int kRegsControl = 104;
constexpr int kRegsSoftmax = 200;
// P_t reaches the MMA warp in two pieces (keys [0, 96) and [96, 128)), each on its own barrier.
constexpr unsigned kPublishMask = 0xC;
__host__ __device__ constexpr int piece_of_chunk(int c) {
  int n = 0;
  for (int i = 0; i < c; ++i) n += (kPublishMask >> i) & 1u;
  return n;
}

struct PersistParams {
  int s;
  int bh;
  int num_qblocks;
  int num_items;
  int causal;
  float scale_log2;
  int bh_offset;
  int num_dst;
  int first_dst;
};
struct PersistOutMaps {
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
// Bounded wait of this kernel: a dozen instructions per site (the general mbar_wait, with its
// clock arithmetic, is four times that, and this kernel has two dozen wait sites that all count
// against the instruction cache).  The bound is a poll count: every 4096 polls the status word is
// looked at, and after 2^22 polls (each try_wait itself blocks for a while, so this is seconds,
// not milliseconds) the wait gives up, records the site and lets every role unwind.
constexpr uint32_t kPollLimit = 1u << 22;
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, int* status, int site) {
#pragma unroll 1
  for (uint32_t polls = 1; !mbar_try_wait(bar, parity); ++polls) {
    if ((polls & 0xfffu) == 0 && (*reinterpret_cast<volatile int*>(status) != 0 || polls >= kPollLimit)) {
      atomicOr(status, SILE_ERR_TIMEOUT | (1 << (8 + (site & 15))));
      return false;
    }
  }
  return true;
}
template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

__device__ __forceinline__ int kv_blocks_for_tile(const PersistParams& p, int q0) {
  if (q0 >= p.s) return 0;
  const int all = (p.s + kBlockKV - 1) / kBlockKV;
  if (!p.causal) return all;
  const int last_q = min(q0 + kTileQ, p.s) - 1;
  return min(all, last_q / kBlockKV + 1);
}

// Work item -> (batch*head, query block).  Heads are taken in groups of kHeadGroup; inside a group
// the late query blocks (heavy under a causal mask) of every head come first.  CTAs that run at
// the same time then share the K / V of a few heads in L2, and the items handed out last are the
// light ones.  Not inlined: it runs once per item and role, and its integer divisions would
// otherwise sit in the middle of the hot loops' instruction stream.
struct WorkItem {
  int bh, q_base, n0, n1;
};
__device__ __noinline__ WorkItem decode_item(int item, int bh_total, int num_qblocks, int s, int causal) {
  constexpr int kHeadGroup = 8;
  PersistParams p{};
  p.s = s;
  p.causal = causal;
  const int group = item / (kHeadGroup * num_qblocks);
  const int in_group = item - group * kHeadGroup * num_qblocks;
  const int heads_here = min(kHeadGroup, bh_total - group * kHeadGroup);
  WorkItem w;
  w.bh = group * kHeadGroup + in_group % heads_here;
  w.q_base = (num_qblocks - 1 - in_group / heads_here) * kBlockQ;
  w.n0 = kv_blocks_for_tile(p, w.q_base);
  w.n1 = kv_blocks_for_tile(p, w.q_base + kTileQ);
  return w;
}

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_persistent_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                           const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ PersistOutMaps out_maps,
                           const PersistParams p, int* __restrict__ status, int* __restrict__ work_counter) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemBar);
  uint64_t* q_full = bars;            // [2] Q tile t loaded
  uint64_t* q_empty = bars + 2;       // [2] last Q_t K^T of the item finished
  uint64_t* k_full = bars + 4;        // [2]
  uint64_t* k_empty = bars + 6;       // [2]
  uint64_t* v_full = bars + 8;        // [2]
  uint64_t* v_empty = bars + 10;      // [2]
  uint64_t* s_full = bars + 12;       // [2] S_t written by the tensor core
  uint64_t* p_full = bars + 14;       // [2][4] piece c of P_t written by the softmax warps
  uint64_t* o_done = bars + 22;       // [2] last O_t += P_t V_j of the item finished
  uint64_t* sched_full = bars + 24;   // [kRing]
  uint64_t* sched_empty = bars + 28;  // [kRing]
  volatile int* ring = reinterpret_cast<volatile int*>(bars + 32);  // [kRing]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 34);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tma_q);
    prefetch_tensormap(&tma_k);
    prefetch_tensormap(&tma_v);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&o_done[i], 1);
    }
    for (int i = 0; i < 8; ++i) mbar_init(&p_full[i], 4);  // one arrival per softmax warp of the tile
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&sched_full[i], 1);
      mbar_init(&sched_empty[i], 9);  // the MMA warp and the 8 softmax warps
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
  const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_o[2] = {tmem_base + 256, tmem_base + 384};

  // Item at queue position k of this CTA: the item index, -1 when the queue is exhausted, -2 when
  // a wait ran out.  Every lane of a consuming warp reads the slot; one arrival per warp.
  auto fetch_warp = [&](uint32_t& k) -> int {
    const int slot = k & (kRing - 1);
    const bool w = wait_bar(&sched_full[slot], (k / kRing) & 1, status, 10);
    if (!__all_sync(0xffffffffu, w)) return -2;
    const int item = ring[slot];
    __syncwarp();
    if (lane == 0) mbar_arrive(&sched_empty[slot]);
    ++k;
    return item;
  };

  if (warp < 4) {
    reg_dec<kRegsControl>();
    if (warp == 0) {
      // ---------------- TMA producer and scheduler ----------------
      if (lane == 0) {
        bool ok = true;
        uint32_t g = 0;            // K / V blocks loaded so far (all items)
        uint32_t ic[2] = {0, 0};   // items so far in which tile t had work
        // The next item is drawn while the last blocks of the current one load, late enough that
        // items stay with the counter -- and so with whichever CTA is free first -- as long as
        // possible (drawing further ahead leaves some CTAs holding unstarted heavy items at the
        // end while others idle), early enough that the MMA warp, which runs two blocks behind
        // this lane, finds the position published when it needs it for the item boundary.
        uint32_t pub = 0;  // queue positions published so far
        auto publish = [&](int item) {
          const int slot = pub & (kRing - 1);
          if (!wait_bar(&sched_empty[slot], ((pub / kRing) & 1) ^ 1u, status, 11)) return false;
          ring[slot] = item;
          mbar_arrive(&sched_full[slot]);
          ++pub;
          return true;
        };
        auto draw = [&]() {
          const int item = atomicAdd(work_counter, 1);
          return item < p.num_items ? item : -1;
        };
        int cur = draw();
        ok = publish(cur);
        while (cur >= 0 && ok) {
          const WorkItem w = decode_item(cur, p.bh, p.num_qblocks, p.s, p.causal);
          const int n_max = max(w.n0, w.n1);
          const int draw_at = max(n_max - 3, 0), publish_at = max(n_max - 2, 0);
          int nxt = -1;
          // One copy of the load code serves Q, K and V: per block the steps are
          // [Q0] K_j [Q1] V_j, the Q tiles with block 0 only.
#pragma unroll 1
          for (int j = 0; j < n_max && ok; ++j, ++g) {
            if (j == draw_at) nxt = draw();
            if (j == publish_at && !publish(nxt)) { ok = false; break; }
            const int st = g & 1;
            const uint32_t ph = (g >> 1) & 1;
#pragma unroll 1
            for (int u = (j == 0 ? 0 : 1); u < 4; u += (j == 0 ? 1 : 2)) {
              const bool is_q = (u & 1) == 0;
              const int t = u >> 1;  // Q tile (u = 0, 2); K (u = 1) or V (u = 3)
              if (is_q && (t == 0 ? w.n0 : w.n1) == 0) continue;
              const CUtensorMap* map = is_q ? &tma_q : (t == 0 ? &tma_k : &tma_v);
              uint8_t* dst = smem + (is_q ? kSmemQ + t * kTileBytes : (t == 0 ? kSmemK : kSmemV) + st * kTileBytes);
              uint64_t* full = is_q ? &q_full[t] : (t == 0 ? &k_full[st] : &v_full[st]);
              uint64_t* empty = is_q ? &q_empty[t] : (t == 0 ? &k_empty[st] : &v_empty[st]);
              const uint32_t parity = is_q ? ((ic[t] & 1) ^ 1u) : (ph ^ 1u);
              const int row0 = is_q ? w.q_base + t * kTileQ : j * kBlockKV;
              if (!wait_bar(empty, parity, status, u)) { ok = false; break; }
              mbar_expect_tx(full, kTileBytes);
              tma_load_3d(dst, map, full, 0, row0, w.bh);
              tma_load_3d(dst + kPanelBytes, map, full, 64, row0, w.bh);
              if (is_q) ++ic[t];
            }
          }
          cur = nxt;
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      // The whole warp runs this loop (waits included) and only the tcgen05 instructions are
      // predicated on one elected lane: see umma_ss_f16_if.
      constexpr uint32_t idesc_s = make_idesc_f16(kTileQ, kBlockKV, true, false, false);  // Q K^T: both K-major
      constexpr uint32_t idesc_o = make_idesc_f16(kTileQ, kD, true, false, true);         // P V: V is MN-major
      const uint32_t q_addr = smem_u32(smem + kSmemQ);
      const uint32_t k_addr = smem_u32(smem + kSmemK);
      const uint32_t v_addr = smem_u32(smem + kSmemV);
      const uint32_t el = elect_one() ? 1u : 0u;
      // Descriptors are built once; inside the unrolled loops only a constant is added to the
      // 14-bit start-address field (a 128 x 128 x 16 MMA runs for 64 cycles: an issue sequence
      // slower than that starves the tensor pipe).
      const uint64_t q_desc[2] = {make_smem_desc_sw128(q_addr, 16, 1024), make_smem_desc_sw128(q_addr + kTileBytes, 16, 1024)};
      const uint64_t k_desc[2] = {make_smem_desc_sw128(k_addr, 16, 1024), make_smem_desc_sw128(k_addr + kTileBytes, 16, 1024)};
      const uint64_t v_desc[2] = {make_smem_desc_sw128(v_addr, kPanelBytes, 1024),
                                  make_smem_desc_sw128(v_addr + kTileBytes, kPanelBytes, 1024)};
      auto wait = [&](uint64_t* bar, uint32_t parity, int site) {
        const bool w = wait_bar(bar, parity, status, site);
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
        // O_t += P_t (TMEM, 8 columns per 16 keys) * V_st (rows = keys, 2048 B per 16 keys; d panels
        // 16 KiB apart), piece by piece as the softmax warps publish P_t
        const uint64_t db = v_desc[st];
        const uint32_t d = tmem_o[t], a = tmem_s[t];
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // 32-key chunks of P, two MMAs each
          if (c == 0 || ((kPublishMask >> (c - 1)) & 1u)) {
            if (!wait(&p_full[t * 4 + piece_of_chunk(c)], parity, 6)) return false;
            tcgen05_fence_after();
          }
#pragma unroll
          for (int kk = 2 * c; kk < 2 * c + 2; ++kk)
            umma_ts_f16_if<1>(el, d, a + kk * 8, db + kk * 128, idesc_o, (accumulate || kk != 0) ? 1u : 0u);
        }
        if (last) umma_commit_if<1>(el, smem_u32(&o_done[t]));
        return true;
      };
      // One loop serves every block of every item.  Per block: P V of tile 0, the tile's next
      // Q K^T, P V of tile 1, its next Q K^T.  "Next" is block j+1 of the item or -- in the slot after
      // the tile's last P V of the item (the item's last block if the tile had no work) -- block 0
      // of the NEXT item, whose Q tile must have arrived.  The kernel's start is the same case:
      // an empty item whose one iteration issues nothing but the first item's first Q K^T.
      bool ok = true;
      uint32_t qk = 0;
      uint32_t g = 0;  // ring index of the current item's K / V block 0
      // bit t of: parity of the S / P hand-offs so far of tile t; parity of its items with work so far
      uint32_t sc_par = 0, ic_par = 0;
      int c0 = 0, c1 = 0;  // block counts of tile 0 / 1 in the current item
      while (ok) {
        const int n_max = max(c0, c1);
        const int iters = max(n_max, 1);
        const uint32_t g_next = g + n_max;
        const uint32_t par0 = sc_par & 1u, par1 = (sc_par >> 1) & 1u;
        int nxt = -1, x0 = 0, x1 = 0, e0 = -1, e1 = -1;
        bool have_next = false;
        // Blocks whose iteration is far from the item's end (both tiles have this block and the
        // two after it) run in a loop of their own with nothing but waits, MMAs and commits:
        // every instruction this warp executes between seeing P and issuing the MMAs, or between
        // the MMAs and the commit that wakes the softmax warps, is on the chain that bounds the
        // kernel, and the conditions of the general loop below cost 6 % when every block pays them.
        const int hot_end = (c0 > 0 && c1 > 0) ? max(min(c0, c1) - 2, 0) : 0;
        int j = 0;
#pragma unroll 1
        for (; j < hot_end && ok; ++j) {
          const uint32_t bi = g + j;
          const int st = bi & 1;
          const int st_n = (bi + 1) & 1;
          if (!wait(&v_full[st], (bi >> 1) & 1, 5)) { ok = false; break; }
          if (!issue_pv(0, st, (par0 ^ j) & 1u, j > 0, false)) { ok = false; break; }
          if (!wait(&k_full[st_n], ((bi + 1) >> 1) & 1, 4)) { ok = false; break; }
          tcgen05_fence_after();
          issue_s(0, st_n);
          if (!issue_pv(1, st, (par1 ^ j) & 1u, j > 0, false)) { ok = false; break; }
          umma_commit_if<1>(el, smem_u32(&v_empty[st]));
          issue_s(1, st_n);
          umma_commit_if<1>(el, smem_u32(&k_empty[st_n]));
        }
#pragma unroll 1
        for (; j < iters && ok; ++j) {
          const uint32_t bi = g + j;
          const int st = bi & 1;
          const int st_n = (bi + 1) & 1;
          if (n_max > 0 && !wait(&v_full[st], (bi >> 1) & 1, 5)) { ok = false; break; }
          if (!have_next && j >= iters - 2) {
            // The next item is looked up here, not earlier: the producer publishes it while it
            // loads the item's last blocks.
            nxt = fetch_warp(qk);
            if (nxt == -2) { ok = false; break; }
            have_next = true;
            if (nxt >= 0) {
              const WorkItem w = decode_item(nxt, p.bh, p.num_qblocks, p.s, p.causal);
              x0 = w.n0;
              x1 = w.n1;
            }
            e0 = x0 > 0 ? (c0 > 0 ? c0 - 1 : iters - 1) : -1;
            e1 = x1 > 0 ? (c1 > 0 ? c1 - 1 : iters - 1) : -1;
          }
          // ---- tile 0 ----
          if (j < c0) {
            if (!issue_pv(0, st, (par0 ^ j) & 1u, j > 0, j + 1 == c0)) { ok = false; break; }
          }
          {
            const bool in_item = j + 1 < c0;
            if (in_item || j == e0) {
              const uint32_t ki = in_item ? bi + 1 : g_next;
              if (!in_item && !wait(&q_full[0], (ic_par ^ (c0 > 0 ? 1u : 0u)) & 1u, 3)) { ok = false; break; }
              if (!wait(&k_full[ki & 1], (ki >> 1) & 1, 4)) { ok = false; break; }
              tcgen05_fence_after();
              issue_s(0, ki & 1);
              if (in_item ? j + 2 == c0 : x0 == 1) umma_commit_if<1>(el, smem_u32(&q_empty[0]));
            }
          }
          // ---- tile 1 ----
          if (j < c1) {
            if (!issue_pv(1, st, (par1 ^ j) & 1u, j > 0, j + 1 == c1)) { ok = false; break; }
          }
          if (n_max > 0) umma_commit_if<1>(el, smem_u32(&v_empty[st]));
          {
            const bool in_item = j + 1 < c1;
            if (in_item || j == e1) {
              const uint32_t ki = in_item ? bi + 1 : g_next;
              if (!in_item && !wait(&q_full[1], ((ic_par >> 1) ^ (c1 > 0 ? 1u : 0u)) & 1u, 3)) { ok = false; break; }
              if (!wait(&k_full[ki & 1], (ki >> 1) & 1, 4)) { ok = false; break; }
              tcgen05_fence_after();
              issue_s(1, ki & 1);
              if (in_item ? j + 2 == c1 : x1 == 1) umma_commit_if<1>(el, smem_u32(&q_empty[1]));
            }
          }
          if (j + 1 < n_max) umma_commit_if<1>(el, smem_u32(&k_empty[st_n]));
          else if (nxt >= 0) umma_commit_if<1>(el, smem_u32(&k_empty[g_next & 1]));
        }
        if (nxt < 0) break;
        g = g_next;
        sc_par ^= (c0 & 1u) | ((c1 & 1u) << 1);
        ic_par ^= (c0 > 0 ? 1u : 0u) | (c1 > 0 ? 2u : 0u);
        c0 = x0;
        c1 = x1;
      }
      __syncwarp();
    }
  } else {
    reg_inc<kRegsSoftmax>();
    // ---------------- softmax / correction / epilogue ----------------
    const int t = (warp - 4) >> 2;        // Q tile of this group of four warps
    const int quarter = warp & 3;         // TMEM lane quarter of this warp
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t ts = tmem_s[t] + lane_off;
    const uint32_t to = tmem_o[t] + lane_off;
    uint8_t* stage = smem + kSmemStage + (warp - 4) * 4096;  // [32 rows][128 B], 1024-byte aligned
    bool ok = true;
    uint32_t qk = 0;
    uint32_t sc = 0;  // S / P hand-offs so far for this tile
    uint32_t ic = 0;  // items so far in which this tile had work

    for (int item = fetch_warp(qk); item >= 0 && ok; item = fetch_warp(qk)) {
      const WorkItem w = decode_item(item, p.bh, p.num_qblocks, p.s, p.causal);
      const int n = t == 0 ? w.n0 : w.n1;
      if (n == 0) continue;
      const int q_tile0 = w.q_base + t * kTileQ;
      const int q_idx = q_tile0 + row_in_tile;
      float m_used = -INFINITY;  // row max (scaled, log2 domain) that P, l and O currently refer to
      float l = 0.0f;

      for (int j = 0; j < n; ++j) {
        if (!wait_bar(&s_full[t], (sc + j) & 1, status, 8)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();

        // A block that needs masking (the diagonal block under a causal mask, a ragged last block)
        // is masked in tensor memory first, 32 keys at a time in a loop that is not unrolled: a
        // round trip of a few hundred cycles on one block in many, instead of two instructions per
        // score unrolled into the loop every block runs through (4 KiB of instruction cache).
        const int kv0 = j * kBlockKV;
        const bool need_mask = (kv0 + kBlockKV > p.s) || (p.causal && kv0 + kBlockKV - 1 > q_tile0);
        if (need_mask) {
          const int limit = p.causal ? min(q_idx, p.s - 1) : p.s - 1;  // last visible key index
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            const int visible = limit - (kv0 + c * 32) + 1;  // of this chunk's 32 keys
            if (__all_sync(0xffffffffu, visible >= 32)) continue;
            uint32_t r[32];
            tmem_ld_32x32b_x32(ts + c * 32, r);
            tcgen05_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i >= visible) r[i] = 0xff800000u;  // -inf
            tmem_st_32x32b_x32(ts + c * 32, r);
          }
          tcgen05_wait_st();
        }
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(ts + c * 32, sr[c]);
        tcgen05_wait_ld();

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
      if (!ok) break;
      sc += n;

      // ---- epilogue of the item ----
      if (!wait_bar(&o_done[t], ic & 1, status, 9)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++ic;
      tcgen05_fence_after();
      // O = acc / l goes out through shared memory, one 64-wide head-dim panel at a time: this
      // warp's 32 rows are converted, written in the 128-byte swizzle into the warp's staging
      // buffer, and lane 0 issues one TMA store per destination.  Global (and NVLink) writes are
      // full 128-byte lines, rows past the end of the sequence are clipped by the tensor map, and
      // with several destinations this is the all-gather of O.
      const float inv_l = 1.0f / l;
      const int row0 = q_tile0 + quarter * 32;
      const uint32_t row_addr = smem_u32(stage) + lane * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {  // 32 head-dim columns at a time; two of them fill a panel
        uint32_t orow[32];
        tmem_ld_32x32b_x32(to + c * 32, orow);
        tcgen05_wait_ld();
        if ((c & 1) == 0) {
          if (lane == 0) tma_store_wait_read<0>();  // the previous panel has left the staging buffer
          __syncwarp();
        }
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
        if (c & 1) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.s) {
            int d = p.first_dst;
            for (int i = 0; i < p.num_dst; ++i) {
              tma_store_3d(&out_maps.map[d], stage, (c >> 1) * 64, row0, p.bh_offset + w.bh);
              if (++d == p.num_dst) d = 0;
            }
            tma_store_commit();
          }
        }
      }
      // O_t is in registers / on its way out: order the reads before this warp's next P hand-off,
      // which is what lets the next item's first P V overwrite O_t
      tcgen05_fence_before();
      __syncwarp();
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    if (*reinterpret_cast<volatile int*>(status) != 0) {
      // A wait ran out somewhere: give copies and MMAs still in flight time to land before
      // tensor memory is released.
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {
      }
    }
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

}  // namespace

// Arguments already validated by attention_launch.
int attention_persistent_launch(const AttnProblem& a, cudaStream_t stream) {
  int* status = nullptr;
  if (int rc = device_status_word(&status)) return rc;
  int* counter = nullptr;
  if (int rc = device_work_counter(&counter)) return rc;

  CUtensorMap tq, tk, tv;
  const uint64_t dims[3] = {static_cast<uint64_t>(kD), static_cast<uint64_t>(a.s), static_cast<uint64_t>(a.bh)};
  const uint64_t strides[2] = {static_cast<uint64_t>(kD) * 2, static_cast<uint64_t>(a.s) * kD * 2};
  const uint32_t box[3] = {64, 128, 1};
  if (int rc = encode_tensor_map(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = encode_tensor_map(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.k, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = encode_tensor_map(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.v, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;

  PersistParams p{};
  p.s = static_cast<int>(a.s);
  p.bh = static_cast<int>(a.bh);
  p.num_qblocks = static_cast<int>((a.s + kBlockQ - 1) / kBlockQ);
  const int64_t items = static_cast<int64_t>(p.bh) * p.num_qblocks;
  if (items > 0x3fffffffll) return fail(SILE_ERR_INVALID, "attention: too many blocks");
  p.num_items = static_cast<int>(items);
  p.causal = a.causal ? 1 : 0;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.bh_offset = static_cast<int>(a.num_peers > 0 ? a.bh_offset : 0);
  p.num_dst = a.num_peers > 0 ? a.num_peers : 1;
  p.first_dst = a.num_peers > 0 ? a.peer_first : 0;

  PersistOutMaps out_maps;
  {
    const uint64_t bh_total = static_cast<uint64_t>(a.num_peers > 0 ? a.bh_total : a.bh);
    const uint64_t odims[3] = {static_cast<uint64_t>(kD), static_cast<uint64_t>(a.s), bh_total};
    const uint32_t obox[3] = {64, 32, 1};  // one staged panel: 64 head-dim columns x a warp's 32 rows
    for (int i = 0; i < p.num_dst; ++i) {
      void* base = a.num_peers > 0 ? a.peer_o[i] : a.o;
      if (int rc = encode_tensor_map(&out_maps.map[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, odims, strides, obox, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    }
    for (int i = p.num_dst; i < 8; ++i) out_maps.map[i] = out_maps.map[0];
  }

  static bool attr_set[kMaxDevices] = {};
  static int sm_count[kMaxDevices] = {};
  const int slot = current_device_slot();
  if (!attr_set[slot]) {
    SILE_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    int dev = 0, sms = 0;
    SILE_CUDA_TRY(cudaGetDevice(&dev));
    SILE_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    sm_count[slot] = sms;
    attr_set[slot] = true;
  }
  // The queue starts at zero for every launch; the counter is this launch's own (see
  // device_work_counter), reset in stream order just before the kernel.
  SILE_CUDA_TRY(cudaMemsetAsync(counter, 0, sizeof(int), stream));
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(items, sm_count[slot]));  // one persistent CTA per SM
  attn_fwd_persistent_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tq, tk, tv, out_maps, p, status, counter);
  SILE_CUDA_TRY(cudaGetLastError());
  note_kernel("attn_fwd_persistent_kernel", grid, kThreads, kSmemBytes);
  return SILE_OK;
}

}  // namespace sile
