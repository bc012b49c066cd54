/*
 * CPU oracle for the sile tile-kernel hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of what sile's CPU backend generates and runs for the
 * GEMM / softmax / reduction / elementwise example kernels, plus the attention
 * forward composed from the same tile ops.  It exists to check the CUDA
 * kernels; nothing in the product path may call it.
 *
 * Pinning: the GEMM, vec_add, relu, softmax and parallel_reduce functions are
 * checked against the golden vectors of the reference's own tests
 * (crates/sile/tests/backend_matmul.rs:29-64, llvm_ir_cpu_runtime.rs:53-140,
 * backend_vec_add.rs:15-24, backend_softmax.rs:21-37,
 * backend_parallel_reduce.rs:16-28).  The reference has no attention kernel
 * and no attention test, so the attention function here is PARITY UNPINNED:
 * it follows the reference's per-op arithmetic but no reference vector exists.
 */
#ifndef SILE_ORACLE_H
#define SILE_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Tile sizes the reference bakes into generated code from const generics
 * (crates/sile-tile-ir/src/lower.rs:9-34).  The exact-ABI entry points below
 * read them from here.  Not thread safe; tests set them before each call. */
void sile_oracle_bind_matmul(int64_t bm, int64_t bn, int64_t bk);
void sile_oracle_bind_vec_add(int64_t tile);
void sile_oracle_bind_softmax(int64_t bm, int64_t bn);
void sile_oracle_bind_parallel_reduce(int64_t tile);
void sile_oracle_bind_matvec(int64_t bm, int64_t bk);

/* Exact C ABI of the generated wrappers
 * (crates/sile-backend/src/cpu/codegen.rs:433-555; Rust side cpu/mod.rs:12,
 * 104-128): buffers in kernel-parameter order, shapes = concatenation of
 * every argument's shape. */
void sile_kernel_matmul(void** buffers, int64_t num_threadgroups,
                        int64_t threads_per_group, const int64_t* shapes,
                        int64_t num_shapes);
void sile_kernel_vec_add(void** buffers, int64_t num_threadgroups,
                         int64_t threads_per_group, const int64_t* shapes,
                         int64_t num_shapes);
void sile_kernel_relu(void** buffers, int64_t num_threadgroups,
                      int64_t threads_per_group, const int64_t* shapes,
                      int64_t num_shapes);
void sile_kernel_softmax(void** buffers, int64_t num_threadgroups,
                         int64_t threads_per_group, const int64_t* shapes,
                         int64_t num_shapes);
void sile_kernel_parallel_reduce(void** buffers, int64_t num_threadgroups,
                                 int64_t threads_per_group,
                                 const int64_t* shapes, int64_t num_shapes);
void sile_kernel_matvec(void** buffers, int64_t num_threadgroups,
                        int64_t threads_per_group, const int64_t* shapes,
                        int64_t num_shapes);

/* Canonical matmul with explicit tile sizes; only the listed logical tiles
 * (row-major tile ids, pid = ti * (N/BN) + tj) are computed when tile_ids is
 * non-NULL -- the sampled form used for sizes the scalar path cannot finish.
 * Follows canonical_matmul.rs:128-444. */
void sile_oracle_matmul(const float* a, const float* b, float* c, int64_t m,
                        int64_t n, int64_t k, int64_t bm, int64_t bn,
                        int64_t bk, int64_t num_threadgroups);
void sile_oracle_matmul_tiles(const float* a, const float* b, float* c,
                              int64_t m, int64_t n, int64_t k, int64_t bm,
                              int64_t bn, int64_t bk, const int64_t* tile_ids,
                              int64_t num_tiles);

/* Matmul whose accumulator is seeded with the output tile, C = C + A*B through the general
 * tile mma (tile_compute/mma.rs:25-260) -- the path the reference takes when the canonical
 * pattern does not match.  c is read and written in place. */
void sile_oracle_matmul_acc(const float* a, const float* b, float* c, int64_t m,
                            int64_t n, int64_t k, int64_t bm, int64_t bn,
                            int64_t bk, int64_t num_threadgroups);

/* Attention forward composed from the reference's tile ops (general mma path,
 * left-fold reductions, expf).  q,o: [bh*s, d]; kt: [bh*d, s] (K supplied
 * transposed, the DSL has no transpose op); v: [bh*s, d]; all f32 row-major.
 * One logical tile = (bh index, q-tile of bm rows); units lists
 * bh_index * (s/bm) + q_tile, or NULL for all.  PARITY UNPINNED. */
void sile_oracle_attention(const float* q, const float* kt, const float* v,
                           float* o, int64_t bh, int64_t s, int64_t d,
                           int64_t bm, int64_t bn, float scale, int causal,
                           const int64_t* units, int64_t num_units);

int sile_oracle_num_threads(void);
void sile_oracle_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
