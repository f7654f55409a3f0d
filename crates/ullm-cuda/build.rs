// Builds or finds libullm_cuda.
//
//  * ULLM_CUDA_LIB_DIR set: link the prebuilt shared library found there
//    (`python -m ullm_b200.build` writes ullm_b200/libullm_cuda.so).
//  * otherwise ULLM_CUDA_SRC_DIR (default: ../../ullm_b200/csrc relative to this crate) is compiled
//    with nvcc through the `cc` crate, for sm_100a only: no other architecture, no CPU fallback.
use std::{env, path::PathBuf};

fn main() {
    println!("cargo:rerun-if-env-changed=ULLM_CUDA_LIB_DIR");
    println!("cargo:rerun-if-env-changed=ULLM_CUDA_SRC_DIR");
    if let Ok(dir) = env::var("ULLM_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-lib=dylib=ullm_cuda");
        return;
    }
    let src = env::var("ULLM_CUDA_SRC_DIR")
        .map(PathBuf::from)
        .unwrap_or_else(|_| PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../ullm_b200/csrc"));
    let mut build = cc::Build::new();
    build
        .cuda(true)
        .cudart("static")
        .flag("-gencode")
        .flag("arch=compute_100a,code=sm_100a")
        .flag("-std=c++17")
        .flag("-O3")
        .flag("-lineinfo")
        .flag("--expt-relaxed-constexpr");
    for entry in std::fs::read_dir(&src).expect("ULLM_CUDA_SRC_DIR is not a directory") {
        let path = entry.unwrap().path();
        if path.extension().map(|e| e == "cu").unwrap_or(false) {
            println!("cargo:rerun-if-changed={}", path.display());
            build.file(path);
        }
    }
    build.compile("ullm_cuda");
    println!("cargo:rustc-link-lib=dylib=dl");
}
