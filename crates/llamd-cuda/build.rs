//! Build the CUDA kernels when a CUDA toolkit is present; a stub otherwise.
//!
//! Same contract as `llamd-rocm/build.rs`: the workspace must build on a machine without the toolkit, so a missing
//! `nvcc` is reported as a warning and the crate is compiled without `cfg(cuda)`; every wrapper then answers
//! `Error::unsupported`. NOT COMPILED where these sources were written (no Rust toolchain there): the library itself
//! is built and tested through the same `nvcc` command line by `llamd_rs_b200/build.py`.
//!
//! The kernels are written for one target, sm_100a (B200). `LLAMD_CUDA_ARCH` overrides the architecture pair for
//! experiments; `--fmad=false` is NOT optional: the kernels reproduce the CPU path's separate multiply and add.

use std::path::{Path, PathBuf};
use std::process::Command;

fn main() {
    println!("cargo::rerun-if-changed=../../llamd_rs_b200/csrc");
    println!("cargo::rerun-if-changed=../../include");
    println!("cargo::rerun-if-env-changed=CUDA_PATH");
    println!("cargo::rerun-if-env-changed=LLAMD_CUDA_ARCH");
    println!("cargo::rustc-check-cfg=cfg(cuda)");

    let cuda = std::env::var("CUDA_PATH").unwrap_or_else(|_| "/usr/local/cuda".into());
    let nvcc = Path::new(&cuda).join("bin/nvcc");
    if !nvcc.is_file() {
        println!("cargo::warning=nvcc not found under {cuda}; llamd-cuda builds as a stub");
        return;
    }
    let arch = std::env::var("LLAMD_CUDA_ARCH").unwrap_or_else(|_| "arch=compute_100a,code=sm_100a".into());
    let csrc = PathBuf::from(std::env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../llamd_rs_b200/csrc");
    let out_dir = PathBuf::from(std::env::var("OUT_DIR").unwrap());

    let mut sources: Vec<PathBuf> = match std::fs::read_dir(&csrc) {
        Ok(rd) => rd
            .filter_map(|e| e.ok().map(|e| e.path()))
            .filter(|p| matches!(p.extension().and_then(|x| x.to_str()), Some("cu") | Some("cpp")))
            .collect(),
        Err(_) => {
            println!("cargo::warning=kernel sources not found at {}; llamd-cuda builds as a stub", csrc.display());
            return;
        }
    };
    sources.sort();

    let lib = out_dir.join("libllamd_cuda_kernels.a");
    let _ = std::fs::remove_file(&lib); // `ar crs` would keep objects of files that no longer exist
    let mut objs = Vec::new();
    for src in &sources {
        let obj = out_dir.join(format!("{}.o", src.file_name().unwrap().to_string_lossy()));
        let ok = Command::new(&nvcc)
            .args(["-gencode", &arch, "-O3", "-lineinfo", "-std=c++17", "--fmad=false", "-Xcompiler", "-fPIC", "-c"])
            .arg(src)
            .arg("-o")
            .arg(&obj)
            .status()
            .map(|s| s.success())
            .unwrap_or(false);
        if !ok {
            println!("cargo::warning=nvcc failed on {}; llamd-cuda builds as a stub", src.display());
            return;
        }
        objs.push(obj);
    }
    let archived = Command::new("ar").arg("crs").arg(&lib).args(&objs).status().map(|s| s.success()).unwrap_or(false);
    if !archived {
        println!("cargo::warning=ar failed; llamd-cuda builds as a stub");
        return;
    }
    println!("cargo::rustc-link-search=native={}", out_dir.display());
    println!("cargo::rustc-link-lib=static=llamd_cuda_kernels");
    println!("cargo::rustc-link-search=native={cuda}/lib64");
    println!("cargo::rustc-link-lib=dylib=cudart");
    println!("cargo::rustc-link-lib=dylib=stdc++");
    println!("cargo::rustc-link-lib=dylib=dl"); // NCCL is opened with dlopen, only when expert parallelism is used
    println!("cargo::rustc-link-arg=-Wl,-rpath,{cuda}/lib64");
    println!("cargo::rustc-cfg=cuda");
    println!("cargo::warning=llamd-cuda: kernels built for {arch}");
}
