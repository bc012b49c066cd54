// build.rs for sile-backend with the `cuda` feature: produces libsile_cuda.so for sm_100a and
// links it.  NOT COMPILED in the environment this file was written in (no Rust toolchain).
//
// Inputs (environment):
//   SILE_CUDA_LIB_DIR   directory holding a prebuilt libsile_cuda.so; skips the nvcc step
//   SILE_CUDA_SRC_DIR   directory with the library's sources (api.cu, gemm_sm100.cu,
//                       attn_sm100.cu, attn_persist_sm100.cu, attn_pair_sm100.cu, tileops.cu,
//                       internal.h, ptx.cuh); default: ../../sile_b200/csrc next to this crate
//   CUDA_HOME           toolkit root (default /usr/local/cuda)
use std::env;
use std::path::PathBuf;
use std::process::Command;

const SOURCES: [&str; 6] = [
    "api.cu",
    "gemm_sm100.cu",
    "attn_sm100.cu",
    "attn_persist_sm100.cu",
    "attn_pair_sm100.cu",
    "tileops.cu",
];

fn main() {
    if env::var_os("CARGO_FEATURE_CUDA").is_none() {
        return;
    }
    println!("cargo:rerun-if-env-changed=SILE_CUDA_LIB_DIR");
    println!("cargo:rerun-if-env-changed=SILE_CUDA_SRC_DIR");

    let lib_dir = if let Some(dir) = env::var_os("SILE_CUDA_LIB_DIR") {
        PathBuf::from(dir)
    } else {
        let src_dir = env::var_os("SILE_CUDA_SRC_DIR")
            .map(PathBuf::from)
            .unwrap_or_else(|| PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../sile_b200/csrc"));
        let out_dir = PathBuf::from(env::var("OUT_DIR").unwrap());
        let cuda_home = env::var("CUDA_HOME").unwrap_or_else(|_| "/usr/local/cuda".to_string());
        let nvcc = PathBuf::from(&cuda_home).join("bin/nvcc");
        let mut cmd = Command::new(nvcc);
        // the same line sile_b200/build.py runs: sm_100a only, no other arch, no fallback
        cmd.args(["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC"]);
        cmd.arg("-o").arg(out_dir.join("libsile_cuda.so"));
        for s in SOURCES {
            let path = src_dir.join(s);
            println!("cargo:rerun-if-changed={}", path.display());
            cmd.arg(path);
        }
        for h in ["internal.h", "ptx.cuh"] {
            println!("cargo:rerun-if-changed={}", src_dir.join(h).display());
        }
        let status = cmd.status().expect("failed to run nvcc");
        assert!(status.success(), "nvcc failed building libsile_cuda.so");
        out_dir
    };
    println!("cargo:rustc-link-search=native={}", lib_dir.display());
    println!("cargo:rustc-link-lib=dylib=sile_cuda");
    // the CUDA runtime is linked into the .so; at run time the loader must find libsile_cuda.so
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", lib_dir.display());
}
