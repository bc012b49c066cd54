//! CUDA backend for sile over libsile_cuda.so (C ABI: include/sile_cuda.h).
//!
//! NOT COMPILED in the environment this file was written in (no Rust toolchain); written against
//! the C header and the types of sile-core / sile-hir.
//!
//! Shaped after the one GPU backend the project has, `MetalBackend::execute_llir(func,
//! param_kinds, args, launch, stream)` (crates/sile-backend/src/metal/mod.rs:65-76), with one
//! difference: the kernels are hand-written for sm_100a, so nothing is generated from the
//! LLVM-like IR.  The backend looks at the kernel's HIR body, decides which library kernel
//! serves it (`recognise`, the analogue of `CanonicalMatmulPlan::detect`,
//! crates/sile-tile-ir/src/passes/lowering/canonical_matmul.rs:446-666) and launches that; a body
//! it does not recognise is `Error::UnsupportedBackend`, which is what every kernel gets on
//! `Device::Cuda` today (crates/sile/src/kernel_launcher.rs:69-71).
//!
//! Like the Metal backend this one stages host tensors per launch (`Tensor` is a host `Vec<f32>`,
//! crates/sile/src/tensor.rs:5-9): `sile_cuda_launch_host` copies inputs in, runs, copies the
//! output back and returns when complete, so `Stream::synchronize` may stay a no-op.  With a
//! device-resident `Tensor` the same descriptor goes to `sile_cuda_launch` with device pointers.

mod recognise;

use std::ffi::{c_char, c_int, c_void, CStr};

use sile_core::{Error, KernelArg, LaunchConfig, Result, Stream};
use sile_hir::Kernel;

pub use recognise::recognise;

pub const SILE_OP_MATMUL: i32 = 1;
pub const SILE_OP_ATTENTION: i32 = 2;
pub const SILE_OP_VEC_ADD: i32 = 3;
pub const SILE_OP_RELU: i32 = 4;
pub const SILE_OP_SOFTMAX: i32 = 5;
pub const SILE_OP_PARALLEL_REDUCE: i32 = 6;
pub const SILE_OP_MATVEC: i32 = 7;
pub const SILE_DTYPE_F32: i32 = 0;
pub const SILE_LAYOUT_ROW_MAJOR: i32 = 0;
pub const SILE_FLAG_ACCUMULATE: i32 = 1;

/// `SileKernelDesc` of include/sile_cuda.h.
#[repr(C)]
#[derive(Clone, Copy, Debug, PartialEq)]
pub struct SileKernelDesc {
    pub struct_size: u32,
    pub op: i32,
    pub in_dtype: i32,
    pub out_dtype: i32,
    pub b_layout: i32,
    pub causal: i32,
    pub scale: f32,
    pub flags: i32,
    pub consts: [i64; 4],
}

impl SileKernelDesc {
    /// An f32, row-major descriptor: the only element type and layout the HIR can express
    /// (crates/sile-hir/src/types.rs:11-14; crates/sile-tile-ir/src/lower.rs:991-1002).
    pub fn f32(op: i32, consts: &[i64]) -> Self {
        let mut c = [0i64; 4];
        c[..consts.len()].copy_from_slice(consts);
        Self {
            struct_size: std::mem::size_of::<Self>() as u32,
            op,
            in_dtype: SILE_DTYPE_F32,
            out_dtype: SILE_DTYPE_F32,
            b_layout: SILE_LAYOUT_ROW_MAJOR,
            causal: 0,
            scale: 1.0,
            flags: 0,
            consts: c,
        }
    }
}

extern "C" {
    fn sile_cuda_device_count() -> c_int;
    fn sile_cuda_set_device(index: c_int) -> c_int;
    fn sile_cuda_launch_host(
        desc: *const SileKernelDesc,
        host_buffers: *const *mut c_void,
        shapes: *const i64,
        num_shapes: i64,
        grid: *const u32,
    ) -> c_int;
    fn sile_cuda_last_error() -> *const c_char;
}

pub struct CudaBackend;

impl CudaBackend {
    pub fn new() -> Result<Self> {
        if unsafe { sile_cuda_device_count() } < 1 {
            return Err(Error::UnsupportedBackend("no CUDA device found"));
        }
        check(unsafe { sile_cuda_set_device(0) })?;
        Ok(Self)
    }

    /// Launch `kernel` over host tensors.  Buffers and shapes are gathered exactly as the CPU
    /// runtime gathers them for `sile_kernel_<name>` (crates/sile-backend/src/cpu/mod.rs:104-107);
    /// only the product of the grid matters, as there (cpu/mod.rs:109-120).
    pub fn execute_hir(
        &self,
        kernel: &Kernel,
        args: &[KernelArg<'_>],
        launch: &LaunchConfig,
        _stream: &Stream,
    ) -> Result<()> {
        let desc = recognise(kernel)?;
        let buffers: Vec<*mut c_void> = args.iter().map(|a| a.mut_ptr as *mut c_void).collect();
        let shapes: Vec<i64> = args.iter().flat_map(|a| a.shape.iter().copied()).collect();
        check(unsafe {
            sile_cuda_launch_host(&desc, buffers.as_ptr(), shapes.as_ptr(), shapes.len() as i64, launch.grid.as_ptr())
        })
    }
}

/// Status codes of include/sile_cuda.h onto `sile_core::Error`
/// (crates/sile-core/src/error.rs:2-13).
fn check(rc: c_int) -> Result<()> {
    if rc == 0 {
        return Ok(());
    }
    let message = unsafe { CStr::from_ptr(sile_cuda_last_error()) }.to_string_lossy().into_owned();
    Err(match rc {
        1 => Error::Shape(message),                                   // SILE_ERR_INVALID
        2 => Error::UnsupportedBackend("kernel or shape not served by libsile_cuda"), // SILE_ERR_UNSUPPORTED
        5 => Error::InvalidDevice(message),                           // SILE_ERR_NO_DEVICE
        _ => Error::Compile(message),                                 // SILE_ERR_CUDA, SILE_ERR_TIMEOUT: run-time failure
    })
}
