//! `build.rs` of a generated project whose GPU backend is CUDA: compiles the library from
//! the sources the generator copied to `csrc/` and `include/` (the command
//! `aot-llm_b200/build.py` runs) and links it. Needs `nvcc` (CUDA 12.8 or later) on PATH.
//! Not compiled where it was written (no Rust toolchain there).
use std::path::PathBuf;
use std::process::Command;

fn main() {
    if std::env::var("CARGO_FEATURE_CUDA").is_err() {
        return;
    }
    let out = PathBuf::from(std::env::var("OUT_DIR").expect("OUT_DIR"));
    let lib = out.join("libaot_cuda.so");
    let nvcc = std::env::var("NVCC").unwrap_or_else(|_| "nvcc".into());
    // --fmad=false and -ffp-contract=off are load-bearing: the CPU kernels never contract
    // a*b+c, and the library reproduces their f32 results bit for bit.
    let status = Command::new(&nvcc)
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--fmad=false"])
        .args(["-Xcompiler", "-fPIC,-ffp-contract=off,-O2", "-shared", "-Iinclude"])
        .arg("-o")
        .arg(&lib)
        .arg("csrc/aotcu.cu")
        .status()
        .unwrap_or_else(|e| panic!("cannot run {nvcc}: {e}"));
    assert!(status.success(), "nvcc failed");
    for f in ["csrc", "include"] {
        println!("cargo:rerun-if-changed={f}");
    }
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=aot_cuda");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", out.display());
}
