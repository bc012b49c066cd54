// C++ mirror of the reference's kernel description (sile_hir::Kernel) and the recogniser that
// maps such a description onto libsile_cuda's kernels.
//
// In the reference a `#[sile::kernel]` body becomes a `sile_hir::Kernel` value
// (crates/sile-hir/src/kernel.rs:40-83: name, const parameters, tensor parameters and a list of
// Let / Assign / Store / AtomicAdd / ForLoop statements over Builtin expressions) which every
// backend then compiles.  A CUDA backend that owns hand-written kernels cannot compile arbitrary
// bodies; it has to decide, from the body's STRUCTURE, whether a kernel is one it can serve.
// `sile::recognise` is that decision: it resolves let-bound names, compares the body with the
// patterns below and returns the SileKernelDesc to launch, or throws
// Error(UnsupportedBackend), the outcome the reference's own Cuda arm has today
// (crates/sile/src/kernel_launcher.rs:69-71).  Names (of the kernel, its parameters and its
// locals) play no part in the match.
//
// Patterns, each the HIR the reference's macro front end (crates/sile-macros/src/frontend/
// lower.rs:140-400) produces for the example of that name:
//   matmul           crates/sile/examples/matmul.rs:3-18, mlp.rs:6-22; detection mirrors what
//                    CanonicalMatmulPlan::detect requires of the tile IR
//                    (crates/sile-tile-ir/src/passes/lowering/canonical_matmul.rs:446-666).
//                    The same body with the accumulator seeded from the output tile
//                    (`let mut acc = c.load_tile([BM, BN], [pid0, pid1])`) is the reference's
//                    general `mma(a, b, acc)` (tile_compute/mma.rs:25-260) and maps to the
//                    matmul with SILE_FLAG_ACCUMULATE; any other seed is refused
//   vec_add          crates/sile/examples/vec_add.rs:3-13
//   relu             crates/sile/examples/mlp.rs:51-55
//   softmax          crates/sile/examples/softmax.rs:3-16
//   parallel_reduce  crates/sile/examples/parallel_reduce.rs:3-9
//   matvec           crates/sile/examples/mlp.rs:28-46
// The fused attention kernel has no HIR form (the DSL has neither a transpose nor an index tile for
// the causal mask); it is reached through SILE_OP_ATTENTION descriptors only.
#ifndef SILE_HIR_HPP
#define SILE_HIR_HPP

#include <cmath>
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "sile.hpp"

namespace sile {
namespace hir {

// crates/sile-hir/src/kernel.rs:3-31
enum class ParamKind { Input, Output };
enum class BuiltinOp {
  ProgramId, LoadTile, LoadTileLike2D, Store, Max, Add, Sub, Mul, Div, Exp, ReduceMax, ReduceSum,
  Reshape, Broadcast, ShapeOf, Mma, Constant, ScalarDiv, ShapeDim, Index
};

// crates/sile-hir/src/types.rs:3-9
struct ShapeExpr {
  enum class Kind { Dynamic, Constant, Symbol, Tuple };
  Kind kind = Kind::Dynamic;
  int64_t value = 0;
  std::string name;
  std::vector<ShapeExpr> dims;
  static ShapeExpr dynamic() { return ShapeExpr{}; }
  static ShapeExpr constant(int64_t v) {
    ShapeExpr s;
    s.kind = Kind::Constant;
    s.value = v;
    return s;
  }
  static ShapeExpr symbol(std::string n) {
    ShapeExpr s;
    s.kind = Kind::Symbol;
    s.name = std::move(n);
    return s;
  }
  static ShapeExpr tuple(std::vector<ShapeExpr> d) {
    ShapeExpr s;
    s.kind = Kind::Tuple;
    s.dims = std::move(d);
    return s;
  }
  size_t rank() const { return kind == Kind::Tuple ? dims.size() : 1; }  // types.rs:45-50
};

enum class ElemType { F32 };  // types.rs:11-14
struct Type {                 // types.rs:24-30
  enum class Kind { Tensor, Tile, Shape, Scalar };
  Kind kind = Kind::Tensor;
  ElemType elem = ElemType::F32;
  ShapeExpr shape;
  static Type tensor(ElemType e, ShapeExpr s) { return Type{Kind::Tensor, e, std::move(s)}; }
  static Type tile(ElemType e, ShapeExpr s) { return Type{Kind::Tile, e, std::move(s)}; }
};

struct Param {  // kernel.rs:33-38
  std::string name;
  ParamKind kind;
  Type ty;
};

struct Expr {  // kernel.rs:75-82
  enum class Kind { Var, Shape, ScalarI64, ScalarF32, Builtin };
  Kind kind = Kind::ScalarI64;
  std::string var;
  ShapeExpr shape;
  int64_t i = 0;
  float f = 0.0f;
  BuiltinOp op = BuiltinOp::ProgramId;
  std::vector<Expr> args;
  static Expr Var(std::string n) {
    Expr e;
    e.kind = Kind::Var;
    e.var = std::move(n);
    return e;
  }
  static Expr Shape(ShapeExpr s) {
    Expr e;
    e.kind = Kind::Shape;
    e.shape = std::move(s);
    return e;
  }
  static Expr ScalarI64(int64_t v) {
    Expr e;
    e.kind = Kind::ScalarI64;
    e.i = v;
    return e;
  }
  static Expr ScalarF32(float v) {
    Expr e;
    e.kind = Kind::ScalarF32;
    e.f = v;
    return e;
  }
  static Expr Builtin(BuiltinOp op, std::vector<Expr> args = {}) {
    Expr e;
    e.kind = Kind::Builtin;
    e.op = op;
    e.args = std::move(args);
    return e;
  }
};

struct Stmt {  // kernel.rs:48-73
  enum class Kind { Let, Assign, Store, AtomicAdd, ForLoop };
  Kind kind = Kind::Let;
  std::string name;  // Let / Assign: the variable; Store / AtomicAdd: the target; ForLoop: the loop variable
  Expr expr;         // Let / Assign: value; Store / AtomicAdd: value; ForLoop: end
  Expr aux;          // AtomicAdd: index; ForLoop: start
  std::vector<Stmt> body;
  static Stmt Let(std::string n, Expr e) { return Stmt{Kind::Let, std::move(n), std::move(e), {}, {}}; }
  static Stmt Assign(std::string n, Expr e) { return Stmt{Kind::Assign, std::move(n), std::move(e), {}, {}}; }
  static Stmt Store(std::string target, Expr v) { return Stmt{Kind::Store, std::move(target), std::move(v), {}, {}}; }
  static Stmt AtomicAdd(std::string target, Expr index, Expr v) {
    return Stmt{Kind::AtomicAdd, std::move(target), std::move(v), std::move(index), {}};
  }
  static Stmt ForLoop(std::string var, Expr start, Expr end, std::vector<Stmt> body) {
    return Stmt{Kind::ForLoop, std::move(var), std::move(end), std::move(start), std::move(body)};
  }
};

struct Kernel {  // kernel.rs:40-46
  std::string name;
  std::vector<std::pair<std::string, int64_t>> const_params;
  std::vector<Param> params;
  std::vector<Stmt> body;
};

}  // namespace hir

namespace detail {

using hir::BuiltinOp;
using hir::Expr;
using hir::ShapeExpr;
using hir::Stmt;

// The body with every let-bound name replaced by its definition; loop variables, parameters and
// loop-carried (assigned) variables stay as Var.
class Resolver {
 public:
  explicit Resolver(const hir::Kernel& k) : kernel_(k) {
    for (const auto& c : k.const_params) consts_[c.first] = c.second;
  }
  void bind(const std::string& name, const Expr& e) { lets_[name] = resolve(e); }
  void keep(const std::string& name) { lets_.erase(name); }

  Expr resolve(const Expr& e) const {
    switch (e.kind) {
      case Expr::Kind::Var: {
        auto it = lets_.find(e.var);
        if (it != lets_.end()) return it->second;
        auto c = consts_.find(e.var);
        if (c != consts_.end()) return Expr::ScalarI64(c->second);
        return e;
      }
      case Expr::Kind::Shape: return Expr::Shape(resolve_shape(e.shape));
      case Expr::Kind::Builtin: {
        Expr out = e;
        for (Expr& a : out.args) a = resolve(a);
        return out;
      }
      default: return e;
    }
  }
  // A shape symbol is a const parameter (-> Constant) or a let-bound scalar expression (kept as a
  // Symbol; expr_of_symbol resolves it).
  ShapeExpr resolve_shape(const ShapeExpr& s) const {
    if (s.kind == ShapeExpr::Kind::Symbol) {
      auto c = consts_.find(s.name);
      if (c != consts_.end()) return ShapeExpr::constant(c->second);
      return s;
    }
    if (s.kind == ShapeExpr::Kind::Tuple) {
      ShapeExpr out = s;
      for (ShapeExpr& d : out.dims) d = resolve_shape(d);
      return out;
    }
    return s;
  }
  Expr expr_of_symbol(const ShapeExpr& s) const {
    if (s.kind == ShapeExpr::Kind::Constant) return Expr::ScalarI64(s.value);
    if (s.kind == ShapeExpr::Kind::Symbol) return resolve(Expr::Var(s.name));
    return Expr::Shape(s);
  }
  int param_index(const std::string& name) const {
    for (size_t i = 0; i < kernel_.params.size(); ++i)
      if (kernel_.params[i].name == name) return static_cast<int>(i);
    return -1;
  }

 private:
  const hir::Kernel& kernel_;
  std::map<std::string, Expr> lets_;
  std::map<std::string, int64_t> consts_;
};

inline bool is_op(const Expr& e, BuiltinOp op, size_t nargs) {
  return e.kind == Expr::Kind::Builtin && e.op == op && e.args.size() == nargs;
}
inline bool is_var(const Expr& e, const std::string& name) { return e.kind == Expr::Kind::Var && e.var == name; }
inline bool is_i64(const Expr& e, int64_t v) { return e.kind == Expr::Kind::ScalarI64 && e.i == v; }
inline bool is_zero_f32(const Expr& e) {
  return (e.kind == Expr::Kind::ScalarF32 && e.f == 0.0f) || (e.kind == Expr::Kind::ScalarI64 && e.i == 0);
}
// tile::id().d  ==  ShapeDim(ProgramId, d)
inline bool is_program_id(const Expr& e, int64_t d) {
  return is_op(e, BuiltinOp::ShapeDim, 2) && is_op(e.args[0], BuiltinOp::ProgramId, 0) && is_i64(e.args[1], d);
}
// t.shape()[d]  ==  ShapeDim(Var(t), d)  or  ShapeDim(ShapeOf(Var(t)), d)
inline bool is_shape_dim_of(const Expr& e, const std::string& tensor, int64_t d) {
  if (!is_op(e, BuiltinOp::ShapeDim, 2) || !is_i64(e.args[1], d)) return false;
  const Expr& t = e.args[0];
  return is_var(t, tensor) || (is_op(t, BuiltinOp::ShapeOf, 1) && is_var(t.args[0], tensor));
}
// A constant shape [d0, d1, ...] -> its extents
inline bool const_dims(const Expr& e, size_t rank, int64_t* out) {
  if (e.kind != Expr::Kind::Shape) return false;
  const ShapeExpr& s = e.shape;
  if (rank == 1 && s.kind == ShapeExpr::Kind::Constant) {
    out[0] = s.value;
    return true;
  }
  if (s.kind != ShapeExpr::Kind::Tuple || s.dims.size() != rank) return false;
  for (size_t i = 0; i < rank; ++i) {
    if (s.dims[i].kind != ShapeExpr::Kind::Constant || s.dims[i].value <= 0) return false;
    out[i] = s.dims[i].value;
  }
  return true;
}

struct TileLoad {
  std::string tensor;
  std::vector<int64_t> dims;
  std::vector<Expr> coords;
};
// LoadTile(Var(tensor), Shape([dims]), Shape([coords]))
inline bool match_load(const Resolver& r, const Expr& e, size_t rank, TileLoad* out) {
  if (!is_op(e, BuiltinOp::LoadTile, 3) || e.args[0].kind != Expr::Kind::Var) return false;
  out->tensor = e.args[0].var;
  out->dims.assign(rank, 0);
  if (!const_dims(e.args[1], rank, out->dims.data())) return false;
  if (e.args[2].kind != Expr::Kind::Shape) return false;
  const ShapeExpr& c = e.args[2].shape;
  out->coords.clear();
  if (c.kind == ShapeExpr::Kind::Tuple) {
    if (c.dims.size() != rank) return false;
    for (const ShapeExpr& d : c.dims) out->coords.push_back(r.expr_of_symbol(d));
  } else {
    if (rank != 1) return false;
    out->coords.push_back(r.expr_of_symbol(c));
  }
  return true;
}

inline SileKernelDesc make_desc(int op, std::initializer_list<int64_t> consts) { return f32_desc(op, consts); }

inline bool tensor_rank_is(const hir::Param& p, size_t rank) {
  return p.ty.kind == hir::Type::Kind::Tensor && p.ty.elem == hir::ElemType::F32 && p.ty.shape.rank() == rank;
}

// Reads the straight-line prefix of `body` into the resolver; returns the index of the first
// statement that is not a Let.
inline size_t bind_lets(Resolver& r, const std::vector<Stmt>& body, size_t from = 0) {
  size_t i = from;
  for (; i < body.size() && body[i].kind == Stmt::Kind::Let; ++i) r.bind(body[i].name, body[i].expr);
  return i;
}

// for k in 0..(x.shape()[1] / BK)
inline bool match_k_loop(const Resolver& r, const Stmt& loop, const std::string& tensor, int64_t* bk) {
  if (loop.kind != Stmt::Kind::ForLoop || !is_i64(r.resolve(loop.aux), 0)) return false;
  const Expr end = r.resolve(loop.expr);
  if (!(is_op(end, BuiltinOp::Div, 2) || is_op(end, BuiltinOp::ScalarDiv, 2))) return false;
  if (!is_shape_dim_of(end.args[0], tensor, 1) || end.args[1].kind != Expr::Kind::ScalarI64 || end.args[1].i <= 0) return false;
  *bk = end.args[1].i;
  return true;
}

inline bool recognise_matmul(const hir::Kernel& k, SileKernelDesc* out) {
  if (k.params.size() != 3 || k.params[0].kind != hir::ParamKind::Input || k.params[1].kind != hir::ParamKind::Input ||
      k.params[2].kind != hir::ParamKind::Output)
    return false;
  for (const auto& p : k.params)
    if (!tensor_rank_is(p, 2)) return false;
  const std::string &A = k.params[0].name, &B = k.params[1].name, &C = k.params[2].name;
  // find the accumulator: the variable the final Store writes
  if (k.body.size() < 3) return false;
  const Stmt& store = k.body.back();
  if (store.kind != Stmt::Kind::Store || store.name != C || store.expr.kind != Expr::Kind::Var) return false;
  const std::string acc = store.expr.var;
  Resolver r(k);
  const size_t loop_at = bind_lets(r, k.body);
  if (loop_at + 2 != k.body.size()) return false;  // lets, one loop, the store
  // acc = constant(0.0, [BM, BN])  -- the canonical matmul -- or
  // acc = c.load_tile([BM, BN], [pid0, pid1])  -- the accumulator seeded with the output tile,
  // which the reference lowers through its general mma (tile_compute/mma.rs:25-260)
  const Expr acc_init = r.resolve(Expr::Var(acc));
  int64_t bmn[2];
  bool seeded = false;
  if (is_op(acc_init, BuiltinOp::Constant, 2)) {
    if (!is_zero_f32(acc_init.args[0]) || !const_dims(acc_init.args[1], 2, bmn)) return false;
  } else {
    TileLoad lc;
    if (!match_load(r, acc_init, 2, &lc) || lc.tensor != C) return false;
    if (!is_program_id(lc.coords[0], 0) || !is_program_id(lc.coords[1], 1)) return false;
    bmn[0] = lc.dims[0];
    bmn[1] = lc.dims[1];
    seeded = true;
  }
  r.keep(acc);  // loop-carried from here on
  const Stmt& loop = k.body[loop_at];
  int64_t bk = 0;
  if (!match_k_loop(r, loop, A, &bk)) return false;
  r.keep(loop.name);
  const size_t assign_at = bind_lets(r, loop.body);
  if (assign_at + 1 != loop.body.size()) return false;
  const Stmt& upd = loop.body[assign_at];
  if (upd.kind != Stmt::Kind::Assign || upd.name != acc) return false;
  const Expr mma = r.resolve(upd.expr);
  if (!is_op(mma, BuiltinOp::Mma, 3) || !is_var(mma.args[2], acc)) return false;
  TileLoad la, lb;
  if (!match_load(r, mma.args[0], 2, &la) || !match_load(r, mma.args[1], 2, &lb)) return false;
  if (la.tensor != A || lb.tensor != B) return false;
  if (la.dims[0] != bmn[0] || la.dims[1] != bk || lb.dims[0] != bk || lb.dims[1] != bmn[1]) return false;
  if (!is_program_id(la.coords[0], 0) || !is_var(la.coords[1], loop.name)) return false;
  if (!is_var(lb.coords[0], loop.name) || !is_program_id(lb.coords[1], 1)) return false;
  *out = make_desc(SILE_OP_MATMUL, {bmn[0], bmn[1], bk});
  if (seeded) out->flags = SILE_FLAG_ACCUMULATE;
  return true;
}

inline bool recognise_vec_add(const hir::Kernel& k, SileKernelDesc* out) {
  if (k.params.size() != 3 || k.params[2].kind != hir::ParamKind::Output) return false;
  for (const auto& p : k.params)
    if (!tensor_rank_is(p, 1)) return false;
  Resolver r(k);
  const size_t at = bind_lets(r, k.body);
  if (at + 1 != k.body.size()) return false;
  const Stmt& st = k.body[at];
  if (st.kind != Stmt::Kind::Store || st.name != k.params[2].name) return false;
  const Expr v = r.resolve(st.expr);
  if (!is_op(v, BuiltinOp::Add, 2)) return false;
  TileLoad x, y;
  if (!match_load(r, v.args[0], 1, &x) || !match_load(r, v.args[1], 1, &y)) return false;
  const bool direct = x.tensor == k.params[0].name && y.tensor == k.params[1].name;
  const bool swapped = x.tensor == k.params[1].name && y.tensor == k.params[0].name;
  if (!(direct || swapped) || x.dims[0] != y.dims[0]) return false;
  if (!is_program_id(x.coords[0], 0) || !is_program_id(y.coords[0], 0)) return false;
  *out = make_desc(SILE_OP_VEC_ADD, {x.dims[0]});
  return true;
}

inline bool recognise_relu(const hir::Kernel& k, SileKernelDesc* out) {
  if (k.params.size() != 1 || k.params[0].kind != hir::ParamKind::Output || !tensor_rank_is(k.params[0], 1)) return false;
  Resolver r(k);
  const size_t at = bind_lets(r, k.body);
  if (at + 1 != k.body.size()) return false;
  const Stmt& st = k.body[at];
  if (st.kind != Stmt::Kind::Store || st.name != k.params[0].name) return false;
  const Expr v = r.resolve(st.expr);
  if (!is_op(v, BuiltinOp::Max, 2)) return false;
  for (int zero_at = 0; zero_at < 2; ++zero_at) {
    const Expr &z = v.args[zero_at], &d = v.args[1 - zero_at];
    int64_t dz[1];
    TileLoad l;
    if (is_op(z, BuiltinOp::Constant, 2) && is_zero_f32(z.args[0]) && const_dims(z.args[1], 1, dz) && match_load(r, d, 1, &l) &&
        l.tensor == k.params[0].name && l.dims[0] == dz[0] && is_i64(l.coords[0], 0)) {
      *out = make_desc(SILE_OP_RELU, {dz[0]});
      return true;
    }
  }
  return false;
}

// Broadcast(Reshape(v, [BM, 1]), ShapeOf(y))  ->  v
inline bool match_row_broadcast(const Expr& e, const std::string& like, int64_t bm, Expr* inner) {
  if (!is_op(e, BuiltinOp::Broadcast, 2) || !is_op(e.args[0], BuiltinOp::Reshape, 2)) return false;
  const Expr& target = e.args[1];
  if (!(is_op(target, BuiltinOp::ShapeOf, 1) && is_var(target.args[0], like))) {
    int64_t d[2];
    if (!const_dims(target, 2, d) || d[0] != bm) return false;
  }
  int64_t col[2];
  if (!const_dims(e.args[0].args[1], 2, col) || col[0] != bm || col[1] != 1) return false;
  *inner = e.args[0].args[0];
  return true;
}

inline bool same_expr(const Expr& a, const Expr& b);
inline bool same_shape(const ShapeExpr& a, const ShapeExpr& b) {
  if (a.kind != b.kind || a.value != b.value || a.name != b.name || a.dims.size() != b.dims.size()) return false;
  for (size_t i = 0; i < a.dims.size(); ++i)
    if (!same_shape(a.dims[i], b.dims[i])) return false;
  return true;
}
inline bool same_expr(const Expr& a, const Expr& b) {
  if (a.kind != b.kind) return false;
  switch (a.kind) {
    case Expr::Kind::Var: return a.var == b.var;
    case Expr::Kind::Shape: return same_shape(a.shape, b.shape);
    case Expr::Kind::ScalarI64: return a.i == b.i;
    case Expr::Kind::ScalarF32: return a.f == b.f;
    default:
      if (a.op != b.op || a.args.size() != b.args.size()) return false;
      for (size_t i = 0; i < a.args.size(); ++i)
        if (!same_expr(a.args[i], b.args[i])) return false;
      return true;
  }
}

inline bool recognise_softmax(const hir::Kernel& k, SileKernelDesc* out) {
  if (k.params.size() != 2 || k.params[0].kind != hir::ParamKind::Input || k.params[1].kind != hir::ParamKind::Output) return false;
  if (!tensor_rank_is(k.params[0], 2) || !tensor_rank_is(k.params[1], 2)) return false;
  Resolver r(k);
  const std::string &X = k.params[0].name, &Y = k.params[1].name;
  // the output tile's extents are the output parameter's declared shape [BM, BN]
  const ShapeExpr ys = r.resolve_shape(k.params[1].ty.shape);
  int64_t bmn[2];
  if (!const_dims(Expr::Shape(ys), 2, bmn)) return false;
  const size_t at = bind_lets(r, k.body);
  if (at + 1 != k.body.size()) return false;
  const Stmt& st = k.body[at];
  if (st.kind != Stmt::Kind::Store || st.name != Y) return false;
  const Expr v = r.resolve(st.expr);  // num / bcast(reduce_sum(num, 1))
  if (!is_op(v, BuiltinOp::Div, 2)) return false;
  const Expr& num = v.args[0];
  Expr denom;
  if (!match_row_broadcast(v.args[1], Y, bmn[0], &denom)) return false;
  if (!is_op(denom, BuiltinOp::ReduceSum, 2) || !is_i64(denom.args[1], 1) || !same_expr(denom.args[0], num)) return false;
  // num = exp(tile - bcast(reduce_max(tile, 1)))
  if (!is_op(num, BuiltinOp::Exp, 1) || !is_op(num.args[0], BuiltinOp::Sub, 2)) return false;
  const Expr& tile = num.args[0].args[0];
  Expr mx;
  if (!match_row_broadcast(num.args[0].args[1], Y, bmn[0], &mx)) return false;
  if (!is_op(mx, BuiltinOp::ReduceMax, 2) || !is_i64(mx.args[1], 1) || !same_expr(mx.args[0], tile)) return false;
  if (!is_op(tile, BuiltinOp::LoadTileLike2D, 2) || !is_var(tile.args[0], X) || !is_var(tile.args[1], Y)) return false;
  *out = make_desc(SILE_OP_SOFTMAX, {bmn[0], bmn[1]});
  return true;
}

inline bool recognise_parallel_reduce(const hir::Kernel& k, SileKernelDesc* out) {
  if (k.params.size() != 2 || k.params[1].kind != hir::ParamKind::Output) return false;
  if (!tensor_rank_is(k.params[0], 1) || !tensor_rank_is(k.params[1], 1)) return false;
  Resolver r(k);
  const size_t at = bind_lets(r, k.body);
  if (at + 1 != k.body.size()) return false;
  const Stmt& st = k.body[at];
  if (st.kind != Stmt::Kind::AtomicAdd || st.name != k.params[1].name || !is_i64(r.resolve(st.aux), 0)) return false;
  const Expr v = r.resolve(st.expr);  // reduce_sum(load_tile(a, [TILE], [pid]), 0)[0]
  if (!is_op(v, BuiltinOp::Index, 2) || !is_i64(v.args[1], 0)) return false;
  const Expr& sum = v.args[0];
  TileLoad l;
  if (!is_op(sum, BuiltinOp::ReduceSum, 2) || !is_i64(sum.args[1], 0) || !match_load(r, sum.args[0], 1, &l)) return false;
  if (l.tensor != k.params[0].name || !is_program_id(l.coords[0], 0)) return false;
  *out = make_desc(SILE_OP_PARALLEL_REDUCE, {l.dims[0]});
  return true;
}

inline bool recognise_matvec(const hir::Kernel& k, SileKernelDesc* out) {
  if (k.params.size() != 3 || k.params[2].kind != hir::ParamKind::Output) return false;
  if (!tensor_rank_is(k.params[0], 2) || !tensor_rank_is(k.params[1], 1) || !tensor_rank_is(k.params[2], 1)) return false;
  const std::string &X = k.params[0].name, &Y = k.params[1].name, &Z = k.params[2].name;
  if (k.body.size() < 3) return false;
  const Stmt& store = k.body.back();
  if (store.kind != Stmt::Kind::Store || store.name != Z || store.expr.kind != Expr::Kind::Var) return false;
  const std::string acc = store.expr.var;
  Resolver r(k);
  const size_t loop_at = bind_lets(r, k.body);
  if (loop_at + 2 != k.body.size()) return false;
  const Expr acc_init = r.resolve(Expr::Var(acc));
  int64_t bm[1];
  if (!is_op(acc_init, BuiltinOp::Constant, 2) || !is_zero_f32(acc_init.args[0]) || !const_dims(acc_init.args[1], 1, bm)) return false;
  r.keep(acc);
  const Stmt& loop = k.body[loop_at];
  int64_t bk = 0;
  if (!match_k_loop(r, loop, X, &bk)) return false;
  r.keep(loop.name);
  const size_t assign_at = bind_lets(r, loop.body);
  if (assign_at + 1 != loop.body.size()) return false;
  const Stmt& upd = loop.body[assign_at];
  if (upd.kind != Stmt::Kind::Assign || upd.name != acc) return false;
  const Expr add = r.resolve(upd.expr);  // acc + reduce_sum(tile_x * bcast(tile_y), 1)
  if (!is_op(add, BuiltinOp::Add, 2)) return false;
  const int acc_at = is_var(add.args[0], acc) ? 0 : (is_var(add.args[1], acc) ? 1 : -1);
  if (acc_at < 0) return false;
  const Expr& part = add.args[1 - acc_at];
  if (!is_op(part, BuiltinOp::ReduceSum, 2) || !is_i64(part.args[1], 1) || !is_op(part.args[0], BuiltinOp::Mul, 2)) return false;
  for (int x_at = 0; x_at < 2; ++x_at) {
    const Expr &ex = part.args[0].args[x_at], &ey = part.args[0].args[1 - x_at];
    TileLoad lx, ly;
    int64_t bd[2];
    if (!match_load(r, ex, 2, &lx) || lx.tensor != X) continue;
    if (!is_op(ey, BuiltinOp::Broadcast, 2) || !match_load(r, ey.args[0], 1, &ly) || ly.tensor != Y) continue;
    if (!const_dims(ey.args[1], 2, bd)) continue;
    if (lx.dims[0] != bm[0] || lx.dims[1] != bk || ly.dims[0] != bk || bd[0] != bm[0] || bd[1] != bk) continue;
    if (!is_program_id(lx.coords[0], 0) || !is_var(lx.coords[1], loop.name) || !is_var(ly.coords[0], loop.name)) continue;
    *out = make_desc(SILE_OP_MATVEC, {bm[0], bk});
    return true;
  }
  return false;
}

}  // namespace detail

// The descriptor of the library kernel that computes what `kernel` describes; throws
// Error(UnsupportedBackend) when the body matches none of the patterns in this file's header.
inline SileKernelDesc recognise(const hir::Kernel& kernel) {
  SileKernelDesc d{};
  if (detail::recognise_matmul(kernel, &d) || detail::recognise_matvec(kernel, &d) || detail::recognise_vec_add(kernel, &d) ||
      detail::recognise_relu(kernel, &d) || detail::recognise_softmax(kernel, &d) || detail::recognise_parallel_reduce(kernel, &d))
    return d;
  throw Error(Error::Kind::UnsupportedBackend, "kernel '" + kernel.name + "' matches no kernel of libsile_cuda");
}

// KernelLauncher for a described kernel: what `KernelLauncher::new(kernel, args)` is in the
// reference (crates/sile/src/kernel_launcher.rs:15-37), with recognition in place of compilation.
inline KernelLauncher launcher_for(const hir::Kernel& kernel, std::vector<KernelArg> args) {
  return KernelLauncher(recognise(kernel), std::move(args));
}

}  // namespace sile

#endif  // SILE_HIR_HPP
