// Builds libtkv.so with nvcc for sm_100a and links it, the way tempura's kernels crate compiles its C
// with the `cc` crate (kernels/build.rs:1-13).  Source only: not compiled where it was written.
//
// The source list is the one tempura_b200/_build.py builds (SOURCES); tests/test_rust_shim.py keeps the two equal.
use std::{env, path::PathBuf, process::Command};

const SOURCES: &[&str] = &[
    "tkv_lib.cu",
    "tkv_noalloc.cu",
    "tkv_attention.cu",
    "tkv_attention_tc.cu",
    "tkv_prefill_tc.cu",
    "tkv_prefix_index.cu",
    "tkv_hostobj.cpp",
    "tkv_session.cpp",
    "tkv_coordinator.cpp",
];

fn main() {
    // the checkout of the handoff library; by default two levels above this crate
    let root = env::var("TKV_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../..")
    });
    let csrc = root.join("tempura_b200").join("csrc");
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".into());
    let mut cmd = Command::new(nvcc);
    cmd.args([
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        // bit-exact scale arithmetic: no FMA contraction, IEEE division and square root
        "-fmad=false", "-prec-div=true", "-prec-sqrt=true",
        "-Xcompiler", "-fPIC", "-shared", "-o",
    ]);
    cmd.arg(out.join("libtkv.so"));
    for s in SOURCES {
        cmd.arg(csrc.join(s));
        println!("cargo:rerun-if-changed={}", csrc.join(s).display());
    }
    println!("cargo:rerun-if-changed={}", csrc.join("tkv_kernels.cuh").display());
    println!("cargo:rerun-if-changed={}", csrc.join("tkv_attention_tc.h").display());
    println!("cargo:rerun-if-changed={}", csrc.join("tkv_tc_common.cuh").display());
    println!("cargo:rerun-if-changed={}", root.join("include").join("tkv.h").display());
    let status = cmd.status().expect("nvcc not found: set NVCC or put it on PATH");
    assert!(status.success(), "nvcc failed to build libtkv.so");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=tkv");
}
