//! Builds libyscv_cuda.so with nvcc the way crates/yscv-kernels/build.rs drives `cc` for its
//! assembly kernels, or links a prebuilt copy when YSCV_CUDA_LIB_DIR points at one.
use std::{env, path::PathBuf, process::Command};

fn main() {
    println!("cargo:rerun-if-env-changed=YSCV_CUDA_LIB_DIR");
    println!("cargo:rerun-if-env-changed=YSCV_CUDA_SRC");
    if let Ok(dir) = env::var("YSCV_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-lib=dylib=yscv_cuda");
        return;
    }
    // the CUDA sources: yscv_b200/csrc of the library's repository
    let src = PathBuf::from(env::var("YSCV_CUDA_SRC").expect(
        "set YSCV_CUDA_SRC to the library's yscv_b200/csrc directory, or YSCV_CUDA_LIB_DIR to a prebuilt libyscv_cuda.so",
    ));
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let mut sources = Vec::new();
    for entry in std::fs::read_dir(&src).expect("read csrc") {
        let path = entry.unwrap().path();
        if path.extension().map_or(false, |e| e == "cu") {
            println!("cargo:rerun-if-changed={}", path.display());
            sources.push(path);
        }
    }
    sources.sort();
    let lib = out.join("libyscv_cuda.so");
    let status = Command::new(env::var("NVCC").unwrap_or_else(|_| "nvcc".into()))
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo"])
        .args(["-Xcompiler", "-fPIC", "-shared", "-diag-suppress", "177", "-o"])
        .arg(&lib)
        .args(&sources)
        .status()
        .expect("nvcc not found");
    assert!(status.success(), "nvcc failed building libyscv_cuda.so");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=yscv_cuda");
}
