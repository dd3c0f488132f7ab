//! Compiles the CUDA sources of the attention hot path for sm_100a and links them into the crate.
//!
//! SHADY_ATTN_CSRC points at the directory that holds api.cu, append.cu, decode.cu, prefill.cu, p2p.cu and gptq.cu
//! (default: `../../shady_thinker_b200/csrc`, their place in the repository this crate ships in); NVCC
//! overrides the compiler.  There is one target architecture and no other backend.
//!
//! Not compiled where it was written (no Rust toolchain there): reviewed source.
use std::path::PathBuf;
use std::process::Command;

const SOURCES: [&str; 6] = ["api.cu", "append.cu", "decode.cu", "prefill.cu", "p2p.cu", "gptq.cu"];

fn main() {
    let out = PathBuf::from(std::env::var("OUT_DIR").expect("OUT_DIR"));
    let manifest = PathBuf::from(std::env::var("CARGO_MANIFEST_DIR").expect("CARGO_MANIFEST_DIR"));
    let csrc = std::env::var("SHADY_ATTN_CSRC")
        .map(PathBuf::from)
        .unwrap_or_else(|_| manifest.join("../../shady_thinker_b200/csrc"));
    let nvcc = std::env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());
    println!("cargo:rerun-if-env-changed=SHADY_ATTN_CSRC");
    println!("cargo:rerun-if-env-changed=NVCC");
    println!("cargo:rerun-if-changed={}", manifest.join("../../include/shady_attn.h").display());

    let mut objects = Vec::new();
    for src in SOURCES {
        let input = csrc.join(src);
        println!("cargo:rerun-if-changed={}", input.display());
        let object = out.join(src.replace(".cu", ".o"));
        let status = Command::new(&nvcc)
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo"])
            .args(["-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-c"])
            .arg(&input)
            .arg("-o")
            .arg(&object)
            .status()
            .unwrap_or_else(|e| panic!("could not run {nvcc}: {e}"));
        assert!(status.success(), "nvcc failed on {}", input.display());
        objects.push(object);
    }
    let archive = out.join("libshady_attn.a");
    let status = Command::new("ar").arg("crs").arg(&archive).args(&objects).status().expect("ar");
    assert!(status.success(), "ar failed");

    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=static=shady_attn");
    if let Ok(cuda) = std::env::var("CUDA_HOME") {
        println!("cargo:rustc-link-search=native={cuda}/lib64");
    } else {
        println!("cargo:rustc-link-search=native=/usr/local/cuda/lib64");
    }
    println!("cargo:rustc-link-lib=cudart");
    println!("cargo:rustc-link-lib=stdc++");
}
