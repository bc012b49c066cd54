/*
 * CPU oracle for the sile tile-kernel hot path -- TEST INFRASTRUCTURE ONLY.
 * See sile_oracle.h for what is pinned by reference golden vectors and what
 * is not (attention: PARITY UNPINNED).
 *
 * Built with the reference's own flags: cc -shared -fPIC -O2 -fopenmp -lm
 * (crates/sile-backend/src/cpu/mod.rs:83).  On the x86-64 baseline there is
 * no FMA, so "sum + a*b" is a rounded multiply followed by a rounded add, as
 * in the reference's generated C.
 */
#include "sile_oracle.h"

#include <math.h>
#include <omp.h>
#include <stdlib.h>
#include <string.h>

/* Per-thread tile ids, the analogue of the generated prelude's
 * _Thread_local sile_gid_{0,1,2} (cpu/codegen.rs:47-52). */
static _Thread_local int64_t gid0 = 0;
static _Thread_local int64_t gid1 = 0;

static int64_t g_mm_bm = 1, g_mm_bn = 1, g_mm_bk = 1;
static int64_t g_va_tile = 4;
static int64_t g_sm_bm = 1, g_sm_bn = 1;
static int64_t g_pr_tile = 1;
static int64_t g_mv_bm = 1, g_mv_bk = 1;

void sile_oracle_bind_matmul(int64_t bm, int64_t bn, int64_t bk) {
  g_mm_bm = bm; g_mm_bn = bn; g_mm_bk = bk;
}
void sile_oracle_bind_vec_add(int64_t tile) { g_va_tile = tile; }
void sile_oracle_bind_softmax(int64_t bm, int64_t bn) { g_sm_bm = bm; g_sm_bn = bn; }
void sile_oracle_bind_parallel_reduce(int64_t tile) { g_pr_tile = tile; }
void sile_oracle_bind_matvec(int64_t bm, int64_t bk) { g_mv_bm = bm; g_mv_bk = bk; }

int sile_oracle_num_threads(void) { return omp_get_max_threads(); }
/* The reference's runtime leaves the thread count to OpenMP's default (all cores); a launcher
 * that exports OMP_NUM_THREADS=1 to its children would otherwise pin the baseline to one core. */
void sile_oracle_set_num_threads(int n) { if (n > 0) omp_set_num_threads(n); }

/* ---- GEMM: canonical whole-kernel pattern ------------------------------- */

/* One output tile.  canonical_matmul.rs:128-444: rows outer, cols inner,
 * sum starts at 0.0f, k runs 0 .. (K/BK)*BK strictly in order, A walked with
 * unit stride and B with stride ldb, one store per element. */
static void matmul_tile(const float* a, const float* b, float* c, int64_t n,
                        int64_t k, int64_t bm, int64_t bn, int64_t bk,
                        int64_t pid0, int64_t pid1) {
  const int64_t lda = k, ldb = n, ldc = n;
  const int64_t k_limit = (k / bk) * bk; /* lower.rs:214-444: trip count K/BK */
  const int64_t c_tile_base = pid0 * bm * ldc + pid1 * bn;
  for (int64_t row = 0; row < bm; ++row) {
    for (int64_t col = 0; col < bn; ++col) {
      float sum = 0.0f;
      int64_t ai = (pid0 * bm + row) * lda;
      int64_t bi = pid1 * bn + col;
      for (int64_t kk = 0; kk < k_limit; ++kk) {
        sum = sum + a[ai] * b[bi];
        ai += 1;
        bi += ldb;
      }
      c[c_tile_base + row * ldc + col] = sum;
    }
  }
}

/* Wrapper semantics, cpu/codegen.rs:409-431,517-551: the grid collapses to
 * its product; tile coordinates come from the OUTPUT shape; pids past the
 * tile count do nothing. */
void sile_oracle_matmul(const float* a, const float* b, float* c, int64_t m,
                        int64_t n, int64_t k, int64_t bm, int64_t bn,
                        int64_t bk, int64_t num_threadgroups) {
  const int64_t tiles_n = n / bn;
  const int64_t total_tiles = (m / bm) * tiles_n;
#pragma omp parallel for schedule(static)
  for (int64_t tg = 0; tg < num_threadgroups; ++tg) {
    int64_t pid = tg;
    if (pid < total_tiles) {
      gid0 = pid / tiles_n;
      gid1 = pid % tiles_n;
      matmul_tile(a, b, c, n, k, bm, bn, bk, gid0, gid1);
    }
  }
}

void sile_oracle_matmul_tiles(const float* a, const float* b, float* c,
                              int64_t m, int64_t n, int64_t k, int64_t bm,
                              int64_t bn, int64_t bk, const int64_t* tile_ids,
                              int64_t num_tiles) {
  const int64_t tiles_n = n / bn;
  const int64_t total_tiles = (m / bm) * tiles_n;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t i = 0; i < num_tiles; ++i) {
    int64_t pid = tile_ids ? tile_ids[i] : i;
    if (pid >= 0 && pid < total_tiles)
      matmul_tile(a, b, c, n, k, bm, bn, bk, pid / tiles_n, pid % tiles_n);
  }
}

void sile_kernel_matmul(void** buffers, int64_t num_threadgroups,
                        int64_t threads_per_group, const int64_t* shapes,
                        int64_t num_shapes) {
  (void)num_shapes;
  /* shapes = [M,K, K,N, M,N] (cpu/mod.rs:107) */
  const float* a = (const float*)buffers[0];
  const float* b = (const float*)buffers[1];
  float* c = (float*)buffers[2];
  const int64_t k = shapes[1];
  const int64_t m = shapes[4], n = shapes[5];
  sile_oracle_matmul(a, b, c, m, n, k, g_mm_bm, g_mm_bn, g_mm_bk,
                     num_threadgroups * threads_per_group);
}

/* ---- vec_add: rank-1 pointwise store ------------------------------------ */
/* examples/vec_add.rs:3-10; rank-1 output => total_tiles = shapes[off]
 * (cpu/codegen.rs:415-420), gid0 = pid. */
void sile_kernel_vec_add(void** buffers, int64_t num_threadgroups,
                         int64_t threads_per_group, const int64_t* shapes,
                         int64_t num_shapes) {
  (void)num_shapes;
  const float* a = (const float*)buffers[0];
  const float* b = (const float*)buffers[1];
  float* c = (float*)buffers[2];
  const int64_t total = shapes[2];
  const int64_t t = g_va_tile;
  const int64_t n = num_threadgroups * threads_per_group;
#pragma omp parallel for schedule(static)
  for (int64_t pid = 0; pid < n; ++pid) {
    if (pid < total) {
      for (int64_t i = 0; i < t; ++i)
        c[pid * t + i] = a[pid * t + i] + b[pid * t + i];
    }
  }
}

/* ---- relu via max_tile: select(a >= b, a, b) with a = 0 ------------------ */
/* examples/mlp.rs:51-55; lower.rs:619-641. One tile covers the vector. */
void sile_kernel_relu(void** buffers, int64_t num_threadgroups,
                      int64_t threads_per_group, const int64_t* shapes,
                      int64_t num_shapes) {
  (void)num_shapes;
  float* x = (float*)buffers[0];
  const int64_t d = shapes[0];
  if (num_threadgroups * threads_per_group < 1) return;
  for (int64_t i = 0; i < d; ++i) {
    float zero = 0.0f, v = x[i];
    x[i] = (zero >= v) ? zero : v;
  }
}

/* ---- row softmax --------------------------------------------------------- */
/* examples/softmax.rs:3-16: load tile (pid0,pid1) of [BM,BN]; row max is a
 * left fold starting from element 0 with "next > acc ? next : acc"
 * (tile_compute/reduce.rs:10-31,55-88); num = expf(x - max); denom is a left
 * fold of num; y = num / denom. */
void sile_kernel_softmax(void** buffers, int64_t num_threadgroups,
                         int64_t threads_per_group, const int64_t* shapes,
                         int64_t num_shapes) {
  (void)num_shapes;
  const float* x = (const float*)buffers[0];
  float* y = (float*)buffers[1];
  const int64_t ldx = shapes[1];
  const int64_t rows = shapes[2], cols = shapes[3];
  const int64_t bm = g_sm_bm, bn = g_sm_bn;
  const int64_t tiles_n = cols / bn;
  const int64_t total_tiles = (rows / bm) * tiles_n;
  const int64_t n = num_threadgroups * threads_per_group;
#pragma omp parallel for schedule(static)
  for (int64_t pid = 0; pid < n; ++pid) {
    if (pid >= total_tiles) continue;
    const int64_t p0 = pid / tiles_n, p1 = pid % tiles_n;
    for (int64_t r = 0; r < bm; ++r) {
      const float* xr = x + (p0 * bm + r) * ldx + p1 * bn;
      float* yr = y + (p0 * bm + r) * cols + p1 * bn;
      float mx = xr[0];
      for (int64_t j = 1; j < bn; ++j) {
        float nx = xr[j];
        mx = (nx > mx) ? nx : mx;
      }
      float den = expf(xr[0] - mx);
      for (int64_t j = 1; j < bn; ++j) den = den + expf(xr[j] - mx);
      for (int64_t j = 0; j < bn; ++j) yr[j] = expf(xr[j] - mx) / den;
    }
  }
}

/* ---- parallel_reduce: fused load+sum then atomic add -------------------- */
/* examples/parallel_reduce.rs:3-9.  The from-global sum uses float4 chunks:
 * acc starts 0.0f, acc += (v0+v1+v2+v3) per chunk, then a scalar tail
 * (tile_compute/fused_reduce.rs:1142-1256; helpers cpu/codegen.rs:72-85).
 * The atomic is "#pragma omp atomic update" (cpu/codegen.rs:245-253). */
void sile_kernel_parallel_reduce(void** buffers, int64_t num_threadgroups,
                                 int64_t threads_per_group,
                                 const int64_t* shapes, int64_t num_shapes) {
  (void)num_shapes;
  const float* a = (const float*)buffers[0];
  float* out = (float*)buffers[1];
  /* rank-1 output of extent 1 => total_tiles = extent of the FIRST buffer
   * when no tile plan is inferred (cpu/codegen.rs:487-502). */
  const int64_t total = shapes[0];
  const int64_t t = g_pr_tile;
  const int64_t n = num_threadgroups * threads_per_group;
#pragma omp parallel for schedule(static)
  for (int64_t pid = 0; pid < n; ++pid) {
    if (pid >= total) continue;
    const float* p = a + pid * t;
    float acc = 0.0f;
    int64_t i = 0;
    for (; i + 4 <= t; i += 4) acc = acc + (p[i] + p[i + 1] + p[i + 2] + p[i + 3]);
    for (; i < t; ++i) acc = acc + p[i];
#pragma omp atomic update
    out[0] += acc;
  }
}

/* ---- matvec: fused map-reduce ------------------------------------------- */
/* examples/mlp.rs:28-46: acc[r] = acc[r] + reduce_sum(x_tile * bcast(y_tile),1)
 * per k tile; the map-reduce is a plain left fold from element 0
 * (fused_reduce.rs:189-293). */
void sile_kernel_matvec(void** buffers, int64_t num_threadgroups,
                        int64_t threads_per_group, const int64_t* shapes,
                        int64_t num_shapes) {
  (void)num_shapes;
  const float* x = (const float*)buffers[0];
  const float* y = (const float*)buffers[1];
  float* z = (float*)buffers[2];
  const int64_t k = shapes[1];
  const int64_t total = shapes[3];
  const int64_t bm = g_mv_bm, bk = g_mv_bk;
  const int64_t n = num_threadgroups * threads_per_group;
#pragma omp parallel for schedule(static)
  for (int64_t pid = 0; pid < n; ++pid) {
    if (pid >= total || (pid + 1) * bm > total) continue;
    for (int64_t r = 0; r < bm; ++r) {
      const float* xr = x + (pid * bm + r) * k;
      float acc = 0.0f;
      for (int64_t kt = 0; kt < k / bk; ++kt) {
        float part = xr[kt * bk] * y[kt * bk];
        for (int64_t j = 1; j < bk; ++j)
          part = part + xr[kt * bk + j] * y[kt * bk + j];
        acc = acc + part;
      }
      z[pid * bm + r] = acc;
    }
  }
}

/* ---- attention forward composed from tile ops --------------------------- */
/* General (non-canonical) mma: D = acc + A*B, per (r,c) the sum starts from
 * acc[r][c] and k runs in order (tile_compute/mma.rs:25-260).  Tiles are
 * private float arrays (core/emit/alloc.rs:8-32). */
static void tile_mma(const float* a, int64_t lda, const float* b, int64_t ldb,
                     float* acc, int64_t ldacc, int64_t m, int64_t n,
                     int64_t k) {
  for (int64_t r = 0; r < m; ++r)
    for (int64_t c = 0; c < n; ++c) {
      float sum = acc[r * ldacc + c];
      for (int64_t kk = 0; kk < k; ++kk)
        sum = sum + a[r * lda + kk] * b[kk * ldb + c];
      acc[r * ldacc + c] = sum;
    }
}

/* ---- matmul with the accumulator seeded from the output tile ----------------- */
/* `let mut acc = c.load_tile([BM,BN],[pid0,pid1]); for k { acc = mma(a_k, b_k, acc) }; c.store(acc)`:
 * the seed is not Splat(0), so CanonicalMatmulPlan::detect (canonical_matmul.rs:446-666)
 * refuses the body and every k step runs the general tile mma, whose sums start from acc[r][c]
 * (tile_compute/mma.rs:25-260), on tiles copied into private arrays (tile_memory.rs:22-162). */
void sile_oracle_matmul_acc(const float* a, const float* b, float* c, int64_t m,
                            int64_t n, int64_t k, int64_t bm, int64_t bn,
                            int64_t bk, int64_t num_threadgroups) {
  const int64_t tiles_n = n / bn;
  const int64_t total_tiles = (m / bm) * tiles_n;
#pragma omp parallel for schedule(static)
  for (int64_t tg = 0; tg < num_threadgroups; ++tg) {
    if (tg >= total_tiles) continue;
    const int64_t p0 = tg / tiles_n, p1 = tg % tiles_n;
    float* acc = (float*)malloc(sizeof(float) * bm * bn);
    float* at = (float*)malloc(sizeof(float) * bm * bk);
    float* bt = (float*)malloc(sizeof(float) * bk * bn);
    for (int64_t r = 0; r < bm; ++r)
      for (int64_t cc = 0; cc < bn; ++cc) acc[r * bn + cc] = c[(p0 * bm + r) * n + p1 * bn + cc];
    for (int64_t kt = 0; kt < k / bk; ++kt) {
      for (int64_t r = 0; r < bm; ++r)
        for (int64_t kk = 0; kk < bk; ++kk) at[r * bk + kk] = a[(p0 * bm + r) * k + kt * bk + kk];
      for (int64_t kk = 0; kk < bk; ++kk)
        for (int64_t cc = 0; cc < bn; ++cc) bt[kk * bn + cc] = b[(kt * bk + kk) * n + p1 * bn + cc];
      tile_mma(at, bk, bt, bn, acc, bn, bm, bn, bk);
    }
    for (int64_t r = 0; r < bm; ++r)
      for (int64_t cc = 0; cc < bn; ++cc) c[(p0 * bm + r) * n + p1 * bn + cc] = acc[r * bn + cc];
    free(acc); free(at); free(bt);
  }
}

static void attention_unit(const float* q, const float* kt, const float* v,
                           float* o, int64_t s, int64_t d, int64_t bm,
                           int64_t bn, float scale, int causal, int64_t bhi,
                           int64_t qt) {
  float* st = (float*)malloc(sizeof(float) * bm * bn);
  float* acc = (float*)malloc(sizeof(float) * bm * d);
  float* mrow = (float*)malloc(sizeof(float) * bm);
  float* lrow = (float*)malloc(sizeof(float) * bm);
  const float* qtile = q + (bhi * s + qt * bm) * d;      /* tile_memory.rs:164-228 */
  const float* kbase = kt + bhi * d * s;                 /* [d, s] for this head */
  const float* vbase = v + bhi * s * d;
  for (int64_t r = 0; r < bm; ++r) { mrow[r] = -INFINITY; lrow[r] = 0.0f; }
  for (int64_t i = 0; i < bm * d; ++i) acc[i] = 0.0f;
  const int64_t kv_tiles = s / bn;
  for (int64_t j = 0; j < kv_tiles; ++j) {
    if (causal && j * bn > qt * bm + bm - 1) break;      /* fully masked tile */
    /* S = mma(Q, Kt_j, 0) * scale */
    for (int64_t i = 0; i < bm * bn; ++i) st[i] = 0.0f;
    tile_mma(qtile, d, kbase + j * bn, s, st, bn, bm, bn, d);
    for (int64_t i = 0; i < bm * bn; ++i) st[i] = st[i] * scale;
    if (causal) {
      for (int64_t r = 0; r < bm; ++r)
        for (int64_t c = 0; c < bn; ++c)
          if (j * bn + c > qt * bm + r) st[r * bn + c] = st[r * bn + c] + (-INFINITY);
    }
    for (int64_t r = 0; r < bm; ++r) {
      float* sr = st + r * bn;
      /* reduce_max: left fold from element 0 (reduce.rs:10-31) */
      float mx = sr[0];
      for (int64_t c = 1; c < bn; ++c) { float nx = sr[c]; mx = (nx > mx) ? nx : mx; }
      /* max_tile(m, mx) = (m >= mx) ? m : mx (lower.rs:619-641) */
      float mnew = (mrow[r] >= mx) ? mrow[r] : mx;
      float alpha = expf(mrow[r] - mnew);
      for (int64_t c = 0; c < bn; ++c) sr[c] = expf(sr[c] - mnew);
      float psum = sr[0];
      for (int64_t c = 1; c < bn; ++c) psum = psum + sr[c];
      lrow[r] = lrow[r] * alpha + psum;
      mrow[r] = mnew;
      for (int64_t c = 0; c < d; ++c) acc[r * d + c] = acc[r * d + c] * alpha;
    }
    /* acc = mma(P, V_j, acc * bcast(alpha)) */
    tile_mma(st, bn, vbase + j * bn * d, d, acc, d, bm, d, bn);
  }
  float* otile = o + (bhi * s + qt * bm) * d;
  for (int64_t r = 0; r < bm; ++r)
    for (int64_t c = 0; c < d; ++c) otile[r * d + c] = acc[r * d + c] / lrow[r];
  free(st); free(acc); free(mrow); free(lrow);
}

void sile_oracle_attention(const float* q, const float* kt, const float* v,
                           float* o, int64_t bh, int64_t s, int64_t d,
                           int64_t bm, int64_t bn, float scale, int causal,
                           const int64_t* units, int64_t num_units) {
  const int64_t q_tiles = s / bm;
  const int64_t total = bh * q_tiles;
  const int64_t n = units ? num_units : total;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t i = 0; i < n; ++i) {
    int64_t u = units ? units[i] : i;
    if (u < 0 || u >= total) continue;
    attention_unit(q, kt, v, o, s, d, bm, bn, scale, causal, u / q_tiles,
                   u % q_tiles);
  }
}
