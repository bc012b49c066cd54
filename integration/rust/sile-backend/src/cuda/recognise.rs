//! Which library kernel serves a `#[sile::kernel]` body.
//!
//! NOT COMPILED in the environment this file was written in (no Rust toolchain).  It is a port of
//! `sile::recognise` in include/sile_hir.hpp, which is the form that is built and tested
//! (tests/cpp/recogniser_tests.cpp); when the two disagree, the C++ one is right.
//!
//! A body is matched by STRUCTURE after its let-bound names have been resolved; the names of the
//! kernel, its parameters and its locals play no part.  Patterns are the HIR that the macro front
//! end (crates/sile-macros/src/frontend/lower.rs:140-400) produces for the examples:
//!   matmul            crates/sile/examples/matmul.rs:3-18, mlp.rs:6-22 -- what
//!                     CanonicalMatmulPlan::detect requires of the tile IR
//!                     (crates/sile-tile-ir/src/passes/lowering/canonical_matmul.rs:446-666);
//!                     with the accumulator seeded from the output tile it is the general mma
//!                     (tile_compute/mma.rs:25-260) -> SILE_FLAG_ACCUMULATE
//!   vec_add           crates/sile/examples/vec_add.rs:3-13
//!   relu              crates/sile/examples/mlp.rs:51-55
//!   softmax           crates/sile/examples/softmax.rs:3-16
//!   parallel_reduce   crates/sile/examples/parallel_reduce.rs:3-9
//!   matvec            crates/sile/examples/mlp.rs:28-46

use std::collections::HashMap;

use sile_core::{Error, Result};
use sile_hir::{BuiltinOp, ElemType, Expr, Kernel, Param, ParamKind, ShapeExpr, Stmt, Type};

use super::{
    SileKernelDesc, SILE_FLAG_ACCUMULATE, SILE_OP_MATMUL, SILE_OP_MATVEC, SILE_OP_PARALLEL_REDUCE, SILE_OP_RELU,
    SILE_OP_SOFTMAX, SILE_OP_VEC_ADD,
};

pub fn recognise(kernel: &Kernel) -> Result<SileKernelDesc> {
    matmul(kernel)
        .or_else(|| matvec(kernel))
        .or_else(|| vec_add(kernel))
        .or_else(|| relu(kernel))
        .or_else(|| softmax(kernel))
        .or_else(|| parallel_reduce(kernel))
        .ok_or(Error::UnsupportedBackend("kernel matches no kernel of libsile_cuda"))
}

/// The body with every let-bound name replaced by its definition; loop variables, parameters and
/// loop-carried (assigned) variables stay `Var`.
struct Resolver {
    lets: HashMap<String, Expr>,
    consts: HashMap<String, i64>,
}

impl Resolver {
    fn new(k: &Kernel) -> Self {
        Self { lets: HashMap::new(), consts: k.const_params.iter().cloned().collect() }
    }
    fn bind(&mut self, name: &str, e: &Expr) {
        let r = self.resolve(e);
        self.lets.insert(name.to_string(), r);
    }
    fn keep(&mut self, name: &str) {
        self.lets.remove(name);
    }
    fn resolve(&self, e: &Expr) -> Expr {
        match e {
            Expr::Var(n) => {
                if let Some(d) = self.lets.get(n) {
                    d.clone()
                } else if let Some(c) = self.consts.get(n) {
                    Expr::ScalarI64(*c)
                } else {
                    e.clone()
                }
            }
            Expr::Shape(s) => Expr::Shape(self.resolve_shape(s)),
            Expr::Builtin { op, args } => Expr::Builtin { op: *op, args: args.iter().map(|a| self.resolve(a)).collect() },
            _ => e.clone(),
        }
    }
    fn resolve_shape(&self, s: &ShapeExpr) -> ShapeExpr {
        match s {
            ShapeExpr::Symbol(n) => match self.consts.get(n) {
                Some(c) => ShapeExpr::Constant(*c),
                None => s.clone(),
            },
            ShapeExpr::Tuple(d) => ShapeExpr::Tuple(d.iter().map(|x| self.resolve_shape(x)).collect()),
            _ => s.clone(),
        }
    }
    /// A coordinate written as a shape symbol is a const parameter or a let-bound scalar.
    fn expr_of_symbol(&self, s: &ShapeExpr) -> Expr {
        match s {
            ShapeExpr::Constant(v) => Expr::ScalarI64(*v),
            ShapeExpr::Symbol(n) => self.resolve(&Expr::Var(n.clone())),
            _ => Expr::Shape(s.clone()),
        }
    }
}

fn op_args(e: &Expr, want: BuiltinOp, n: usize) -> Option<&[Expr]> {
    match e {
        Expr::Builtin { op, args } if *op == want && args.len() == n => Some(args),
        _ => None,
    }
}
fn is_var(e: &Expr, name: &str) -> bool {
    matches!(e, Expr::Var(n) if n == name)
}
fn is_i64(e: &Expr, v: i64) -> bool {
    matches!(e, Expr::ScalarI64(x) if *x == v)
}
fn is_zero(e: &Expr) -> bool {
    matches!(e, Expr::ScalarF32(x) if *x == 0.0) || is_i64(e, 0)
}
/// `tile::id().d` == ShapeDim(ProgramId, d)
fn is_program_id(e: &Expr, d: i64) -> bool {
    op_args(e, BuiltinOp::ShapeDim, 2)
        .map(|a| op_args(&a[0], BuiltinOp::ProgramId, 0).is_some() && is_i64(&a[1], d))
        .unwrap_or(false)
}
/// `t.shape()[d]` == ShapeDim(Var(t), d) or ShapeDim(ShapeOf(Var(t)), d)
fn is_shape_dim_of(e: &Expr, tensor: &str, d: i64) -> bool {
    op_args(e, BuiltinOp::ShapeDim, 2)
        .map(|a| {
            is_i64(&a[1], d)
                && (is_var(&a[0], tensor) || op_args(&a[0], BuiltinOp::ShapeOf, 1).map(|s| is_var(&s[0], tensor)).unwrap_or(false))
        })
        .unwrap_or(false)
}
/// A constant shape [d0, d1, ...] -> its extents
fn const_dims(e: &Expr, rank: usize) -> Option<Vec<i64>> {
    let Expr::Shape(s) = e else { return None };
    match s {
        ShapeExpr::Constant(v) if rank == 1 => Some(vec![*v]),
        ShapeExpr::Tuple(d) if d.len() == rank => d
            .iter()
            .map(|x| match x {
                ShapeExpr::Constant(v) if *v > 0 => Some(*v),
                _ => None,
            })
            .collect(),
        _ => None,
    }
}

struct TileLoad {
    tensor: String,
    dims: Vec<i64>,
    coords: Vec<Expr>,
}
/// LoadTile(Var(tensor), Shape([dims]), Shape([coords]))
fn match_load(r: &Resolver, e: &Expr, rank: usize) -> Option<TileLoad> {
    let a = op_args(e, BuiltinOp::LoadTile, 3)?;
    let Expr::Var(tensor) = &a[0] else { return None };
    let dims = const_dims(&a[1], rank)?;
    let Expr::Shape(c) = &a[2] else { return None };
    let coords = match c {
        ShapeExpr::Tuple(d) if d.len() == rank => d.iter().map(|x| r.expr_of_symbol(x)).collect(),
        other if rank == 1 => vec![r.expr_of_symbol(other)],
        _ => return None,
    };
    Some(TileLoad { tensor: tensor.clone(), dims, coords })
}

fn tensor_rank_is(p: &Param, rank: usize) -> bool {
    matches!(&p.ty, Type::Tensor { elem: ElemType::F32, shape } if shape.rank() == rank)
}
/// Binds the straight-line prefix of `body`; returns the index of the first non-Let statement.
fn bind_lets(r: &mut Resolver, body: &[Stmt]) -> usize {
    let mut i = 0;
    while let Some(Stmt::Let { name, expr, .. }) = body.get(i) {
        r.bind(name, expr);
        i += 1;
    }
    i
}
/// `for k in 0..(x.shape()[1] / BK)` -> BK
fn match_k_loop(r: &Resolver, start: &Expr, end: &Expr, tensor: &str) -> Option<i64> {
    if !is_i64(&r.resolve(start), 0) {
        return None;
    }
    let end = r.resolve(end);
    let a = op_args(&end, BuiltinOp::Div, 2).or_else(|| op_args(&end, BuiltinOp::ScalarDiv, 2))?;
    match &a[1] {
        Expr::ScalarI64(bk) if *bk > 0 && is_shape_dim_of(&a[0], tensor, 1) => Some(*bk),
        _ => None,
    }
}

fn matmul(k: &Kernel) -> Option<SileKernelDesc> {
    if k.params.len() != 3
        || k.params[0].kind != ParamKind::Input
        || k.params[1].kind != ParamKind::Input
        || k.params[2].kind != ParamKind::Output
        || !k.params.iter().all(|p| tensor_rank_is(p, 2))
    {
        return None;
    }
    let (a_name, b_name, c_name) = (&k.params[0].name, &k.params[1].name, &k.params[2].name);
    // the accumulator is the variable the final Store writes
    let Some(Stmt::Store { target, value: Expr::Var(acc) }) = k.body.last() else { return None };
    if target != c_name {
        return None;
    }
    let mut r = Resolver::new(k);
    let loop_at = bind_lets(&mut r, &k.body);
    if loop_at + 2 != k.body.len() {
        return None; // lets, one loop, the store
    }
    // acc = constant(0.0, [BM, BN]) -- the canonical matmul -- or
    // acc = c.load_tile([BM, BN], [pid0, pid1]) -- seeded with the output tile
    let acc_init = r.resolve(&Expr::Var(acc.clone()));
    let (bmn, seeded) = if let Some(a) = op_args(&acc_init, BuiltinOp::Constant, 2) {
        if !is_zero(&a[0]) {
            return None;
        }
        (const_dims(&a[1], 2)?, false)
    } else {
        let l = match_load(&r, &acc_init, 2)?;
        if &l.tensor != c_name || !is_program_id(&l.coords[0], 0) || !is_program_id(&l.coords[1], 1) {
            return None;
        }
        (l.dims, true)
    };
    r.keep(acc); // loop-carried from here on
    let Stmt::ForLoop { var, start, end, body } = &k.body[loop_at] else { return None };
    let bk = match_k_loop(&r, start, end, a_name)?;
    r.keep(var);
    let assign_at = bind_lets(&mut r, body);
    if assign_at + 1 != body.len() {
        return None;
    }
    let Stmt::Assign { name, expr } = &body[assign_at] else { return None };
    if name != acc {
        return None;
    }
    let mma = r.resolve(expr);
    let m = op_args(&mma, BuiltinOp::Mma, 3)?;
    if !is_var(&m[2], acc) {
        return None;
    }
    let la = match_load(&r, &m[0], 2)?;
    let lb = match_load(&r, &m[1], 2)?;
    if &la.tensor != a_name || &lb.tensor != b_name {
        return None;
    }
    if la.dims != [bmn[0], bk] || lb.dims != [bk, bmn[1]] {
        return None;
    }
    if !is_program_id(&la.coords[0], 0) || !is_var(&la.coords[1], var) || !is_var(&lb.coords[0], var) || !is_program_id(&lb.coords[1], 1) {
        return None;
    }
    let mut d = SileKernelDesc::f32(SILE_OP_MATMUL, &[bmn[0], bmn[1], bk]);
    if seeded {
        d.flags = SILE_FLAG_ACCUMULATE;
    }
    Some(d)
}

fn vec_add(k: &Kernel) -> Option<SileKernelDesc> {
    if k.params.len() != 3 || k.params[2].kind != ParamKind::Output || !k.params.iter().all(|p| tensor_rank_is(p, 1)) {
        return None;
    }
    let mut r = Resolver::new(k);
    let at = bind_lets(&mut r, &k.body);
    if at + 1 != k.body.len() {
        return None;
    }
    let Stmt::Store { target, value } = &k.body[at] else { return None };
    if target != &k.params[2].name {
        return None;
    }
    let v = r.resolve(value);
    let a = op_args(&v, BuiltinOp::Add, 2)?;
    let x = match_load(&r, &a[0], 1)?;
    let y = match_load(&r, &a[1], 1)?;
    let direct = x.tensor == k.params[0].name && y.tensor == k.params[1].name;
    let swapped = x.tensor == k.params[1].name && y.tensor == k.params[0].name;
    if !(direct || swapped) || x.dims[0] != y.dims[0] || !is_program_id(&x.coords[0], 0) || !is_program_id(&y.coords[0], 0) {
        return None;
    }
    Some(SileKernelDesc::f32(SILE_OP_VEC_ADD, &[x.dims[0]]))
}

fn relu(k: &Kernel) -> Option<SileKernelDesc> {
    if k.params.len() != 1 || k.params[0].kind != ParamKind::Output || !tensor_rank_is(&k.params[0], 1) {
        return None;
    }
    let mut r = Resolver::new(k);
    let at = bind_lets(&mut r, &k.body);
    if at + 1 != k.body.len() {
        return None;
    }
    let Stmt::Store { target, value } = &k.body[at] else { return None };
    if target != &k.params[0].name {
        return None;
    }
    let v = r.resolve(value);
    let a = op_args(&v, BuiltinOp::Max, 2)?;
    for zero_at in 0..2 {
        let (z, d) = (&a[zero_at], &a[1 - zero_at]);
        let Some(c) = op_args(z, BuiltinOp::Constant, 2) else { continue };
        let (Some(dz), Some(l)) = (const_dims(&c[1], 1), match_load(&r, d, 1)) else { continue };
        if is_zero(&c[0]) && l.tensor == k.params[0].name && l.dims[0] == dz[0] && is_i64(&l.coords[0], 0) {
            return Some(SileKernelDesc::f32(SILE_OP_RELU, &[dz[0]]));
        }
    }
    None
}

/// Broadcast(Reshape(v, [BM, 1]), ShapeOf(like) | [BM, _]) -> v
fn match_row_broadcast<'e>(e: &'e Expr, like: &str, bm: i64) -> Option<&'e Expr> {
    let b = op_args(e, BuiltinOp::Broadcast, 2)?;
    let rs = op_args(&b[0], BuiltinOp::Reshape, 2)?;
    let target_ok = op_args(&b[1], BuiltinOp::ShapeOf, 1).map(|s| is_var(&s[0], like)).unwrap_or(false)
        || const_dims(&b[1], 2).map(|d| d[0] == bm).unwrap_or(false);
    let col = const_dims(&rs[1], 2)?;
    if !target_ok || col != [bm, 1] {
        return None;
    }
    Some(&rs[0])
}

fn softmax(k: &Kernel) -> Option<SileKernelDesc> {
    if k.params.len() != 2
        || k.params[0].kind != ParamKind::Input
        || k.params[1].kind != ParamKind::Output
        || !tensor_rank_is(&k.params[0], 2)
        || !tensor_rank_is(&k.params[1], 2)
    {
        return None;
    }
    let mut r = Resolver::new(k);
    let (x_name, y_name) = (&k.params[0].name, &k.params[1].name);
    // the output tile's extents are the output parameter's declared shape [BM, BN]
    let Type::Tensor { shape, .. } = &k.params[1].ty else { return None };
    let bmn = const_dims(&Expr::Shape(r.resolve_shape(shape)), 2)?;
    let at = bind_lets(&mut r, &k.body);
    if at + 1 != k.body.len() {
        return None;
    }
    let Stmt::Store { target, value } = &k.body[at] else { return None };
    if target != y_name {
        return None;
    }
    let v = r.resolve(value); // num / bcast(reduce_sum(num, 1))
    let d = op_args(&v, BuiltinOp::Div, 2)?;
    let num = &d[0];
    let denom = match_row_broadcast(&d[1], y_name, bmn[0])?;
    let ds = op_args(denom, BuiltinOp::ReduceSum, 2)?;
    if !is_i64(&ds[1], 1) || &ds[0] != num {
        return None;
    }
    // num = exp(tile - bcast(reduce_max(tile, 1)))
    let e = op_args(num, BuiltinOp::Exp, 1)?;
    let s = op_args(&e[0], BuiltinOp::Sub, 2)?;
    let tile = &s[0];
    let mx = match_row_broadcast(&s[1], y_name, bmn[0])?;
    let m = op_args(mx, BuiltinOp::ReduceMax, 2)?;
    if !is_i64(&m[1], 1) || &m[0] != tile {
        return None;
    }
    let l = op_args(tile, BuiltinOp::LoadTileLike2D, 2)?;
    if !is_var(&l[0], x_name) || !is_var(&l[1], y_name) {
        return None;
    }
    Some(SileKernelDesc::f32(SILE_OP_SOFTMAX, &[bmn[0], bmn[1]]))
}

fn parallel_reduce(k: &Kernel) -> Option<SileKernelDesc> {
    if k.params.len() != 2 || k.params[1].kind != ParamKind::Output || !k.params.iter().all(|p| tensor_rank_is(p, 1)) {
        return None;
    }
    let mut r = Resolver::new(k);
    let at = bind_lets(&mut r, &k.body);
    if at + 1 != k.body.len() {
        return None;
    }
    let Stmt::AtomicAdd { target, index, value } = &k.body[at] else { return None };
    if target != &k.params[1].name || !is_i64(&r.resolve(index), 0) {
        return None;
    }
    let v = r.resolve(value); // reduce_sum(load_tile(a, [TILE], [pid]), 0)[0]
    let i = op_args(&v, BuiltinOp::Index, 2)?;
    if !is_i64(&i[1], 0) {
        return None;
    }
    let s = op_args(&i[0], BuiltinOp::ReduceSum, 2)?;
    if !is_i64(&s[1], 0) {
        return None;
    }
    let l = match_load(&r, &s[0], 1)?;
    if l.tensor != k.params[0].name || !is_program_id(&l.coords[0], 0) {
        return None;
    }
    Some(SileKernelDesc::f32(SILE_OP_PARALLEL_REDUCE, &[l.dims[0]]))
}

fn matvec(k: &Kernel) -> Option<SileKernelDesc> {
    if k.params.len() != 3
        || k.params[2].kind != ParamKind::Output
        || !tensor_rank_is(&k.params[0], 2)
        || !tensor_rank_is(&k.params[1], 1)
        || !tensor_rank_is(&k.params[2], 1)
    {
        return None;
    }
    let (x_name, y_name, z_name) = (&k.params[0].name, &k.params[1].name, &k.params[2].name);
    let Some(Stmt::Store { target, value: Expr::Var(acc) }) = k.body.last() else { return None };
    if target != z_name {
        return None;
    }
    let mut r = Resolver::new(k);
    let loop_at = bind_lets(&mut r, &k.body);
    if loop_at + 2 != k.body.len() {
        return None;
    }
    let acc_init = r.resolve(&Expr::Var(acc.clone()));
    let c = op_args(&acc_init, BuiltinOp::Constant, 2)?;
    if !is_zero(&c[0]) {
        return None;
    }
    let bm = const_dims(&c[1], 1)?[0];
    r.keep(acc);
    let Stmt::ForLoop { var, start, end, body } = &k.body[loop_at] else { return None };
    let bk = match_k_loop(&r, start, end, x_name)?;
    r.keep(var);
    let assign_at = bind_lets(&mut r, body);
    if assign_at + 1 != body.len() {
        return None;
    }
    let Stmt::Assign { name, expr } = &body[assign_at] else { return None };
    if name != acc {
        return None;
    }
    let add = r.resolve(expr); // acc + reduce_sum(tile_x * bcast(tile_y), 1)
    let a = op_args(&add, BuiltinOp::Add, 2)?;
    let acc_at = if is_var(&a[0], acc) { 0 } else if is_var(&a[1], acc) { 1 } else { return None };
    let part = op_args(&a[1 - acc_at], BuiltinOp::ReduceSum, 2)?;
    if !is_i64(&part[1], 1) {
        return None;
    }
    let mul = op_args(&part[0], BuiltinOp::Mul, 2)?;
    for x_at in 0..2 {
        let (ex, ey) = (&mul[x_at], &mul[1 - x_at]);
        let Some(lx) = match_load(&r, ex, 2) else { continue };
        let Some(b) = op_args(ey, BuiltinOp::Broadcast, 2) else { continue };
        let (Some(ly), Some(bd)) = (match_load(&r, &b[0], 1), const_dims(&b[1], 2)) else { continue };
        if &lx.tensor != x_name || &ly.tensor != y_name || lx.dims != [bm, bk] || ly.dims != [bk] || bd != [bm, bk] {
            continue;
        }
        if !is_program_id(&lx.coords[0], 0) || !is_var(&lx.coords[1], var) || !is_var(&ly.coords[0], var) {
            continue;
        }
        return Some(SileKernelDesc::f32(SILE_OP_MATVEC, &[bm, bk]));
    }
    None
}
