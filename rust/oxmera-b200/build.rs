// NOT COMPILED IN THIS ENVIRONMENT (no Rust toolchain here).
//
// Builds liboxmera_b200.so from the CUDA sources with nvcc, exactly as
// `python -m oxmera_b200.build` does: every translation unit for sm_100a, then
// one shared library.  OXMERA_B200_CSRC points at oxmera_b200/csrc (default:
// ../../oxmera_b200/csrc relative to this crate); OXMERA_B200_LIB_DIR, when set,
// names a directory that already holds a built liboxmera_b200.so and skips nvcc.
use std::env;
use std::path::{Path, PathBuf};
use std::process::Command;

const SOURCES: &[&str] = &[
    "api.cu",
    "gemm_f16_kk.cu",
    "gemm_f16_kn.cu",
    "gemm_f16_mk.cu",
    "gemm_f16_mn.cu",
    "gemm_f8_kk.cu",
    "gemm_f8_kn.cu",
    "gemm_f8_mk.cu",
    "gemm_f8_mn.cu",
    "gemm_tf32.cu",
    "gemm_mx.cu",
];
const ARCH: &[&str] = &["-gencode", "arch=compute_100a,code=sm_100a"];

fn main() {
    println!("cargo:rerun-if-env-changed=OXMERA_B200_LIB_DIR");
    println!("cargo:rerun-if-env-changed=OXMERA_B200_CSRC");
    if let Ok(dir) = env::var("OXMERA_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-lib=dylib=oxmera_b200");
        return;
    }
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").expect("CARGO_MANIFEST_DIR"));
    let csrc = env::var("OXMERA_B200_CSRC")
        .map(PathBuf::from)
        .unwrap_or_else(|_| manifest.join("../../oxmera_b200/csrc"));
    let out = PathBuf::from(env::var("OUT_DIR").expect("OUT_DIR"));
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());

    let mut objects = Vec::new();
    let mut children = Vec::new();
    for src in SOURCES {
        let path = csrc.join(src);
        println!("cargo:rerun-if-changed={}", path.display());
        let obj = out.join(Path::new(src).with_extension("o"));
        let child = Command::new(&nvcc)
            .args(ARCH)
            .args(["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-c"])
            .arg(&path)
            .arg("-o")
            .arg(&obj)
            .spawn()
            .unwrap_or_else(|e| panic!("cannot run {nvcc}: {e}"));
        children.push((src, child));
        objects.push(obj);
    }
    for (src, mut child) in children {
        let status = child.wait().expect("nvcc did not finish");
        assert!(status.success(), "nvcc failed on {src}");
    }
    for header in ["gemm_tcgen05.cuh", "gemm_instances.cuh", "kernels_simt.cuh", "elementwise.cuh", "elem.cuh", "ptx.cuh"] {
        println!("cargo:rerun-if-changed={}", csrc.join(header).display());
    }
    let lib = out.join("liboxmera_b200.so");
    let status = Command::new(&nvcc)
        .args(ARCH)
        .arg("-shared")
        .arg("-o")
        .arg(&lib)
        .args(&objects)
        .status()
        .expect("cannot link");
    assert!(status.success(), "linking liboxmera_b200.so failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=oxmera_b200");
}
