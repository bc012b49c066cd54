// Kernel descriptions (the C++ mirror of sile_hir::Kernel, include/sile_hir.hpp) run through
// sile::recognise.  The descriptions are the ones the reference's tests build by hand
// (crates/sile/tests/llvm_ir_cpu_runtime.rs:143-420) and the HIR its macro front end produces for
// its examples (crates/sile/examples/*.rs; crates/sile-macros/src/frontend/lower.rs:140-400).
//   recogniser_tests            all cases (needs an sm_100 GPU)
//   recogniser_tests --host     recognition only: no device is touched
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "sile_hir.hpp"

using namespace sile;
using hir::BuiltinOp;
using hir::ElemType;
using hir::Expr;
using hir::Kernel;
using hir::Param;
using hir::ParamKind;
using hir::ShapeExpr;
using hir::Stmt;
using hir::Type;

static int failures = 0;
#define CHECK(cond, ...)                                   \
  do {                                                     \
    if (!(cond)) {                                         \
      std::printf("  FAILED %s:%d: ", __FILE__, __LINE__); \
      std::printf(__VA_ARGS__);                            \
      std::printf("\n");                                   \
      ++failures;                                          \
      return;                                              \
    }                                                      \
  } while (0)

static Expr B(BuiltinOp op, std::vector<Expr> args = {}) { return Expr::Builtin(op, std::move(args)); }
static Expr pid(int64_t d) { return B(BuiltinOp::ShapeDim, {B(BuiltinOp::ProgramId), Expr::ScalarI64(d)}); }
static Expr syms(std::vector<const char*> names) {
  std::vector<ShapeExpr> d;
  for (const char* n : names) d.push_back(ShapeExpr::symbol(n));
  return Expr::Shape(ShapeExpr::tuple(d));
}
static Type dyn(size_t rank) {
  if (rank == 1) return Type::tensor(ElemType::F32, ShapeExpr::dynamic());
  return Type::tensor(ElemType::F32, ShapeExpr::tuple(std::vector<ShapeExpr>(rank, ShapeExpr::dynamic())));
}

// llvm_ir_cpu_runtime.rs:143-206 (tile of 4 written as a literal, coordinates through a let)
static Kernel build_vec_add_kernel() {
  Kernel k;
  k.name = "vec_add";
  k.params = {{"a", ParamKind::Input, dyn(1)}, {"b", ParamKind::Input, dyn(1)}, {"c", ParamKind::Output, dyn(1)}};
  const Expr four = Expr::Shape(ShapeExpr::tuple({ShapeExpr::constant(4)}));
  k.body = {Stmt::Let("tid", pid(0)),
            Stmt::Let("x", B(BuiltinOp::LoadTile, {Expr::Var("a"), four, syms({"tid"})})),
            Stmt::Let("y", B(BuiltinOp::LoadTile, {Expr::Var("b"), four, syms({"tid"})})),
            Stmt::Store("c", B(BuiltinOp::Add, {Expr::Var("x"), Expr::Var("y")}))};
  return k;
}

// llvm_ir_cpu_runtime.rs:208-338; `alias_k_tiles` gives the mlp.rs:15-16 form (`let k_tiles = x.shape()[1] / BK`)
static Kernel build_dynamic_k_matmul_kernel(int64_t bm, int64_t bn, int64_t bk, bool alias_k_tiles, const char* name = "matmul") {
  Kernel k;
  k.name = name;
  k.const_params = {{"BM", bm}, {"BN", bn}, {"BK", bk}};
  k.params = {{"a", ParamKind::Input, dyn(2)},
              {"b", ParamKind::Input, dyn(2)},
              {"c", ParamKind::Output, Type::tensor(ElemType::F32, ShapeExpr::tuple({ShapeExpr::symbol("BM"), ShapeExpr::symbol("BN")}))}};
  const Expr trip = B(BuiltinOp::Div, {B(BuiltinOp::ShapeDim, {Expr::Var("a"), Expr::ScalarI64(1)}),
                                       alias_k_tiles ? Expr::Var("BK") : Expr::ScalarI64(bk)});
  k.body = {Stmt::Let("m_idx", pid(0)), Stmt::Let("n_idx", pid(1)),
            Stmt::Let("acc", B(BuiltinOp::Constant, {Expr::ScalarF32(0.0f), syms({"BM", "BN"})}))};
  if (alias_k_tiles) k.body.push_back(Stmt::Let("k_tiles", trip));
  k.body.push_back(Stmt::ForLoop(
      "k_idx", Expr::ScalarI64(0), alias_k_tiles ? Expr::Var("k_tiles") : trip,
      {Stmt::Let("a_tile", B(BuiltinOp::LoadTile, {Expr::Var("a"), syms({"BM", "BK"}), syms({"m_idx", "k_idx"})})),
       Stmt::Let("b_tile", B(BuiltinOp::LoadTile, {Expr::Var("b"), syms({"BK", "BN"}), syms({"k_idx", "n_idx"})})),
       Stmt::Assign("acc", B(BuiltinOp::Mma, {Expr::Var("a_tile"), Expr::Var("b_tile"), Expr::Var("acc")}))}));
  k.body.push_back(Stmt::Store("c", Expr::Var("acc")));
  return k;
}

// llvm_ir_cpu_runtime.rs:340-392
static Kernel build_relu_kernel(int64_t d) {
  Kernel k;
  k.name = "relu";
  k.const_params = {{"D", d}};
  k.params = {{"x", ParamKind::Output, Type::tensor(ElemType::F32, ShapeExpr::tuple({ShapeExpr::symbol("D")}))}};
  k.body = {Stmt::Let("zero", B(BuiltinOp::Constant, {Expr::ScalarF32(0.0f), syms({"D"})})),
            Stmt::Let("data", B(BuiltinOp::LoadTile, {Expr::Var("x"), syms({"D"}), Expr::Shape(ShapeExpr::tuple({ShapeExpr::constant(0)}))})),
            Stmt::Store("x", B(BuiltinOp::Max, {Expr::Var("zero"), Expr::Var("data")}))};
  return k;
}

// examples/softmax.rs:3-16
static Kernel build_softmax_kernel(int64_t bm, int64_t bn) {
  Kernel k;
  k.name = "softmax";
  k.const_params = {{"BM", bm}, {"BN", bn}};
  k.params = {{"x", ParamKind::Input, dyn(2)},
              {"y", ParamKind::Output, Type::tensor(ElemType::F32, ShapeExpr::tuple({ShapeExpr::symbol("BM"), ShapeExpr::symbol("BN")}))}};
  const Expr col = Expr::Shape(ShapeExpr::tuple({ShapeExpr::symbol("BM"), ShapeExpr::constant(1)}));
  const Expr y_shape = B(BuiltinOp::ShapeOf, {Expr::Var("y")});
  k.body = {
      Stmt::Let("tile_x", B(BuiltinOp::LoadTileLike2D, {Expr::Var("x"), Expr::Var("y")})),
      Stmt::Let("tile_x_max", B(BuiltinOp::ReduceMax, {Expr::Var("tile_x"), Expr::ScalarI64(1)})),
      Stmt::Let("tile_x_max_bcast", B(BuiltinOp::Broadcast, {B(BuiltinOp::Reshape, {Expr::Var("tile_x_max"), col}), y_shape})),
      Stmt::Let("num", B(BuiltinOp::Exp, {B(BuiltinOp::Sub, {Expr::Var("tile_x"), Expr::Var("tile_x_max_bcast")})})),
      Stmt::Let("denom", B(BuiltinOp::ReduceSum, {Expr::Var("num"), Expr::ScalarI64(1)})),
      Stmt::Let("denom_bcast", B(BuiltinOp::Broadcast, {B(BuiltinOp::Reshape, {Expr::Var("denom"), col}), y_shape})),
      Stmt::Store("y", B(BuiltinOp::Div, {Expr::Var("num"), Expr::Var("denom_bcast")}))};
  return k;
}

// examples/parallel_reduce.rs:3-9
static Kernel build_parallel_reduce_kernel(int64_t tile) {
  Kernel k;
  k.name = "parallel_reduce";
  k.const_params = {{"TILE", tile}};
  k.params = {{"a", ParamKind::Input, dyn(1)}, {"out", ParamKind::Output, Type::tensor(ElemType::F32, ShapeExpr::tuple({ShapeExpr::constant(1)}))}};
  k.body = {Stmt::Let("pid", pid(0)),
            Stmt::Let("tile_a", B(BuiltinOp::LoadTile, {Expr::Var("a"), syms({"TILE"}), syms({"pid"})})),
            Stmt::Let("sum_tile", B(BuiltinOp::ReduceSum, {Expr::Var("tile_a"), Expr::ScalarI64(0)})),
            Stmt::AtomicAdd("out", Expr::ScalarI64(0), B(BuiltinOp::Index, {Expr::Var("sum_tile"), Expr::ScalarI64(0)}))};
  return k;
}

// examples/mlp.rs:28-46
static Kernel build_matvec_kernel(int64_t bm, int64_t bk) {
  Kernel k;
  k.name = "matvec";
  k.const_params = {{"BM", bm}, {"BK", bk}};
  k.params = {{"x", ParamKind::Input, dyn(2)},
              {"y", ParamKind::Input, dyn(1)},
              {"z", ParamKind::Output, Type::tensor(ElemType::F32, ShapeExpr::tuple({ShapeExpr::symbol("BM")}))}};
  k.body = {Stmt::Let("m_idx", pid(0)),
            Stmt::Let("acc", B(BuiltinOp::Constant, {Expr::ScalarF32(0.0f), syms({"BM"})})),
            Stmt::Let("k_tiles", B(BuiltinOp::Div, {B(BuiltinOp::ShapeDim, {Expr::Var("x"), Expr::ScalarI64(1)}), Expr::Var("BK")})),
            Stmt::ForLoop("k_idx", Expr::ScalarI64(0), Expr::Var("k_tiles"),
                          {Stmt::Let("tile_x", B(BuiltinOp::LoadTile, {Expr::Var("x"), syms({"BM", "BK"}), syms({"m_idx", "k_idx"})})),
                           Stmt::Let("tile_y", B(BuiltinOp::Broadcast, {B(BuiltinOp::LoadTile, {Expr::Var("y"), syms({"BK"}), syms({"k_idx"})}),
                                                                       syms({"BM", "BK"})})),
                           Stmt::Let("partial", B(BuiltinOp::ReduceSum, {B(BuiltinOp::Mul, {Expr::Var("tile_x"), Expr::Var("tile_y")}), Expr::ScalarI64(1)})),
                           Stmt::Assign("acc", B(BuiltinOp::Add, {Expr::Var("acc"), Expr::Var("partial")}))}),
            Stmt::Store("z", Expr::Var("acc"))};
  return k;
}

static bool desc_is(const SileKernelDesc& d, int op, std::vector<int64_t> consts) {
  if (d.op != op || d.in_dtype != SILE_DTYPE_F32 || d.out_dtype != SILE_DTYPE_F32) return false;
  for (size_t i = 0; i < consts.size(); ++i)
    if (d.consts[i] != consts[i]) return false;
  return true;
}

// The matmul body with the accumulator seeded from the output tile: `D = acc + A * B`, the
// reference's general mma (crates/sile-tile-ir/src/passes/lowering/tile_compute/mma.rs:25-260).
static Kernel build_seeded_matmul_kernel(int64_t bm, int64_t bn, int64_t bk) {
  Kernel k = build_dynamic_k_matmul_kernel(bm, bn, bk, false, "matmul_acc");
  k.body[2] = Stmt::Let("acc", B(BuiltinOp::LoadTile, {Expr::Var("c"), syms({"BM", "BN"}), syms({"m_idx", "n_idx"})}));
  return k;
}

// ---- recognition only ------------------------------------------------------------------------
static void recognises_the_reference_examples() {
  {
    const SileKernelDesc d = recognise(build_seeded_matmul_kernel(2, 2, 2));
    CHECK(desc_is(d, SILE_OP_MATMUL, {2, 2, 2}) && d.flags == SILE_FLAG_ACCUMULATE, "matmul with the accumulator seeded from c");
    CHECK(recognise(build_dynamic_k_matmul_kernel(2, 2, 2, false)).flags == 0, "canonical matmul carries no flag");
  }
  CHECK(desc_is(recognise(build_vec_add_kernel()), SILE_OP_VEC_ADD, {4}), "vec_add");
  CHECK(desc_is(recognise(build_dynamic_k_matmul_kernel(2, 2, 2, false)), SILE_OP_MATMUL, {2, 2, 2}), "matmul");
  CHECK(desc_is(recognise(build_dynamic_k_matmul_kernel(32, 16, 8, true, "gemm")), SILE_OP_MATMUL, {32, 16, 8}), "gemm with k_tiles alias");
  CHECK(desc_is(recognise(build_relu_kernel(8)), SILE_OP_RELU, {8}), "relu");
  CHECK(desc_is(recognise(build_softmax_kernel(2, 8)), SILE_OP_SOFTMAX, {2, 8}), "softmax");
  CHECK(desc_is(recognise(build_parallel_reduce_kernel(1000)), SILE_OP_PARALLEL_REDUCE, {1000}), "parallel_reduce");
  CHECK(desc_is(recognise(build_matvec_kernel(32, 8)), SILE_OP_MATVEC, {32, 8}), "matvec");
}

static void names_do_not_matter_structure_does() {
  Kernel k = build_dynamic_k_matmul_kernel(4, 4, 8, true, "whatever");
  CHECK(desc_is(recognise(k), SILE_OP_MATMUL, {4, 4, 8}), "renamed matmul");
  // a kernel CALLED matmul whose body is not the canonical one must be refused
  Kernel sub = build_vec_add_kernel();
  sub.name = "matmul";
  sub.body.back() = Stmt::Store("c", B(BuiltinOp::Sub, {Expr::Var("x"), Expr::Var("y")}));
  bool refused = false;
  try {
    recognise(sub);
  } catch (const Error& e) {
    refused = e.kind() == Error::Kind::UnsupportedBackend && std::string(e.what()).rfind("backend not implemented: ", 0) == 0;
  }
  CHECK(refused, "a - b must be UnsupportedBackend");
}

static void refuses_near_misses() {
  auto refused = [](const Kernel& k) {
    try {
      recognise(k);
    } catch (const Error& e) {
      return e.kind() == Error::Kind::UnsupportedBackend;
    }
    return false;
  };
  {  // B tile indexed [n, k] instead of [k, n]: not the canonical contraction
    Kernel k = build_dynamic_k_matmul_kernel(2, 2, 2, false);
    k.body[3].body[1] = Stmt::Let("b_tile", B(BuiltinOp::LoadTile, {Expr::Var("b"), syms({"BK", "BN"}), syms({"n_idx", "k_idx"})}));
    CHECK(refused(k), "transposed B coordinates");
  }
  {  // accumulator starts at 1.0
    Kernel k = build_dynamic_k_matmul_kernel(2, 2, 2, false);
    k.body[2] = Stmt::Let("acc", B(BuiltinOp::Constant, {Expr::ScalarF32(1.0f), syms({"BM", "BN"})}));
    CHECK(refused(k), "non-zero accumulator");
  }
  {  // accumulator seeded from the A operand's tensor, or from another tile of c
    Kernel k = build_seeded_matmul_kernel(2, 2, 2);
    k.body[2] = Stmt::Let("acc", B(BuiltinOp::LoadTile, {Expr::Var("a"), syms({"BM", "BN"}), syms({"m_idx", "n_idx"})}));
    CHECK(refused(k), "accumulator seeded from a");
    k.body[2] = Stmt::Let("acc", B(BuiltinOp::LoadTile, {Expr::Var("c"), syms({"BM", "BN"}), syms({"n_idx", "m_idx"})}));
    CHECK(refused(k), "accumulator seeded from the transposed tile of c");
  }
  {  // trip count over a.shape()[0]
    Kernel k = build_dynamic_k_matmul_kernel(2, 2, 2, false);
    k.body[3].expr = B(BuiltinOp::Div, {B(BuiltinOp::ShapeDim, {Expr::Var("a"), Expr::ScalarI64(0)}), Expr::ScalarI64(2)});
    CHECK(refused(k), "loop over the wrong dimension");
  }
  {  // softmax without the max subtraction
    Kernel k = build_softmax_kernel(2, 8);
    k.body[3] = Stmt::Let("num", B(BuiltinOp::Exp, {Expr::Var("tile_x")}));
    CHECK(refused(k), "softmax without max subtraction");
  }
  {  // relu against a non-zero constant
    Kernel k = build_relu_kernel(8);
    k.body[0] = Stmt::Let("zero", B(BuiltinOp::Constant, {Expr::ScalarF32(0.5f), syms({"D"})}));
    CHECK(refused(k), "max with 0.5");
  }
  {  // reduction along the wrong axis in matvec
    Kernel k = build_matvec_kernel(32, 8);
    k.body[3].body[2] = Stmt::Let("partial", B(BuiltinOp::ReduceSum, {B(BuiltinOp::Mul, {Expr::Var("tile_x"), Expr::Var("tile_y")}), Expr::ScalarI64(0)}));
    CHECK(refused(k), "matvec reduced along axis 0");
  }
}

// ---- recognised kernels on the device: the reference's golden values ---------------------------
static std::vector<KernelArg> args_of(std::initializer_list<Tensor*> ts) {
  std::vector<KernelArg> a;
  for (Tensor* t : ts) a.push_back(detail::arg(*t));
  return a;
}

// llvm_ir_cpu_runtime.rs:44-103
static void recognised_dynamic_k_matmul_runs() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  Tensor a = Tensor::from_vec({1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16}, {4, 4}, device);
  Tensor b = Tensor::from_vec({1, 0, 2, 1, 0, 1, 3, 2, 1, 0, 4, 3, 0, 1, 5, 4}, {4, 4}, device);
  Tensor c = Tensor::zeros({4, 4}, device);
  launcher_for(build_dynamic_k_matmul_kernel(2, 2, 2, false), args_of({&a, &b, &c})).grid({4, 1, 1}).apply(stream);
  const float expected[16] = {4, 6, 40, 30, 12, 14, 96, 70, 20, 22, 152, 110, 28, 30, 208, 150};
  const std::vector<float> actual = c.to_vec(stream);
  for (int i = 0; i < 16; ++i) CHECK(std::fabs(actual[i] - expected[i]) < 1e-4f, "mismatch at %d: got %f, expected %f", i, actual[i], expected[i]);
}

// The inputs of llvm_ir_cpu_runtime.rs:44-103 with c holding 100 + index before the launch: the
// general mma starts every sum from the accumulator's value, so each output is that seed plus the
// reference test's expected product.
static void recognised_seeded_matmul_runs() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  Tensor a = Tensor::from_vec({1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16}, {4, 4}, device);
  Tensor b = Tensor::from_vec({1, 0, 2, 1, 0, 1, 3, 2, 1, 0, 4, 3, 0, 1, 5, 4}, {4, 4}, device);
  std::vector<float> seed(16);
  for (int i = 0; i < 16; ++i) seed[i] = 100.0f + static_cast<float>(i);
  Tensor c = Tensor::from_vec(seed, {4, 4}, device);
  launcher_for(build_seeded_matmul_kernel(2, 2, 2), args_of({&a, &b, &c})).grid({4, 1, 1}).apply(stream);
  const float product[16] = {4, 6, 40, 30, 12, 14, 96, 70, 20, 22, 152, 110, 28, 30, 208, 150};
  const std::vector<float> actual = c.to_vec(stream);
  for (int i = 0; i < 16; ++i)
    CHECK(std::fabs(actual[i] - (seed[i] + product[i])) < 1e-4f, "mismatch at %d: got %f, expected %f", i, actual[i], seed[i] + product[i]);
  // a short grid leaves the tiles past it with their seed
  Tensor c2 = Tensor::from_vec(seed, {4, 4}, device);
  launcher_for(build_seeded_matmul_kernel(2, 2, 2), args_of({&a, &b, &c2})).grid({3, 1, 1}).apply(stream);
  const std::vector<float> part = c2.to_vec(stream);
  for (int i = 0; i < 16; ++i) {
    const bool last_tile = (i / 4) >= 2 && (i % 4) >= 2;
    const float want = last_tile ? seed[i] : seed[i] + product[i];
    CHECK(std::fabs(part[i] - want) < 1e-4f, "short grid, element %d: got %f, expected %f", i, part[i], want);
  }
}

// llvm_ir_cpu_runtime.rs:8-42 and 105-141
static void recognised_vec_add_and_relu_run() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  Tensor a = Tensor::from_vec(std::vector<float>(16, 1.0f), {16}, device);
  Tensor b = Tensor::from_vec(std::vector<float>(16, 2.0f), {16}, device);
  Tensor c = Tensor::zeros({16}, device);
  launcher_for(build_vec_add_kernel(), args_of({&a, &b, &c})).grid({4, 1, 1}).apply(stream);
  for (float v : c.to_vec(stream)) CHECK(v == 3.0f, "vec_add got %f", v);
  Tensor x = Tensor::from_vec({-3.0f, -1.0f, 0.0f, 2.5f, 4.0f, -7.0f, 8.0f, -0.5f}, {8}, device);
  launcher_for(build_relu_kernel(8), args_of({&x})).grid({1, 1, 1}).apply(stream);
  const float want[8] = {0.0f, 0.0f, 0.0f, 2.5f, 4.0f, 0.0f, 8.0f, 0.0f};
  const std::vector<float> got = x.to_vec(stream);
  for (int i = 0; i < 8; ++i) CHECK(got[i] == want[i], "relu at %d: got %f", i, got[i]);
}

// examples/softmax.rs:18-36, parallel_reduce.rs:11-31, mlp.rs:60-146
static void recognised_softmax_reduce_and_mlp_run() {
  Device device = Device::cuda();
  auto stream = device.create_stream();
  std::vector<float> xs(32);
  for (int i = 0; i < 32; ++i) xs[i] = static_cast<float>(i);
  Tensor x = Tensor::from_vec(xs, {4, 8}, device);
  Tensor y = Tensor::zeros({4, 8}, device);
  launcher_for(build_softmax_kernel(2, 8), args_of({&x, &y})).grid({2, 1, 1}).apply(stream);
  const std::vector<float> p = y.to_vec(stream);
  for (int r = 0; r < 4; ++r) {
    float s = 0.0f;
    for (int c = 0; c < 8; ++c) s += p[r * 8 + c];
    CHECK(std::fabs(s - 1.0f) < 1e-4f, "softmax row %d sums to %f", r, s);
  }
  Tensor a = Tensor::ones({100000}, device);
  Tensor out = Tensor::zeros({1}, device);
  launcher_for(build_parallel_reduce_kernel(1000), args_of({&a, &out})).grid({100, 1, 1}).apply(stream);
  CHECK(std::fabs(out.to_vec(stream)[0] - 100000.0f) < 1e-4f * 100000.0f, "parallel_reduce got %f", out.to_vec(stream)[0]);

  const int64_t n = 64;
  Tensor xin = Tensor::random({n, n}, device), w0 = Tensor::random({n, n}, device), w1 = Tensor::random({n}, device);
  Tensor h = Tensor::zeros({n, n}, device), z = Tensor::zeros({n}, device);
  launcher_for(build_dynamic_k_matmul_kernel(32, 32, 8, true, "gemm"), args_of({&xin, &w0, &h})).grid({2, 2, 1}).apply(stream);
  launcher_for(build_matvec_kernel(32, 8), args_of({&h, &w1, &z})).grid({2, 1, 1}).apply(stream);
  launcher_for(build_relu_kernel(n), args_of({&z})).grid({1, 1, 1}).apply(stream);
  const std::vector<float> hx = xin.to_vec(stream), hw0 = w0.to_vec(stream), hw1 = w1.to_vec(stream), got = z.to_vec(stream);
  for (int64_t r = 0; r < n; ++r) {
    double acc = 0.0;
    for (int64_t c = 0; c < n; ++c) {
      double hrc = 0.0;
      for (int64_t k = 0; k < n; ++k) hrc += static_cast<double>(hx[r * n + k]) * hw0[k * n + c];
      acc += hrc * hw1[c];
    }
    const double want = acc > 0.0 ? acc : 0.0;
    CHECK(std::fabs(got[r] - want) < 1e-3 * (std::fabs(want) + 1.0), "mlp row %lld: got %f, expected %f", (long long)r, got[r], want);
  }
}

int main(int argc, char** argv) {
  const bool host_only = argc > 1 && !std::strcmp(argv[1], "--host");
  struct Case {
    const char* name;
    std::function<void()> fn;
    bool needs_gpu;
  };
  const std::vector<Case> cases = {
      {"recognises_the_reference_examples", recognises_the_reference_examples, false},
      {"names_do_not_matter_structure_does", names_do_not_matter_structure_does, false},
      {"refuses_near_misses", refuses_near_misses, false},
      {"recognised_dynamic_k_matmul_runs", recognised_dynamic_k_matmul_runs, true},
      {"recognised_seeded_matmul_runs", recognised_seeded_matmul_runs, true},
      {"recognised_vec_add_and_relu_run", recognised_vec_add_and_relu_run, true},
      {"recognised_softmax_reduce_and_mlp_run", recognised_softmax_reduce_and_mlp_run, true},
  };
  int ran = 0;
  for (const Case& c : cases) {
    if (host_only && c.needs_gpu) continue;
    const int before = failures;
    std::printf("%s ...\n", c.name);
    try {
      c.fn();
    } catch (const std::exception& e) {
      std::printf("  FAILED with exception: %s\n", e.what());
      ++failures;
    }
    std::printf("%s %s\n", c.name, failures == before ? "ok" : "FAILED");
    ++ran;
  }
  std::printf("%d cases, %d failures\n", ran, failures);
  return failures == 0 ? 0 : 1;
}
