//! Links the TuckCore–CUDA C ABI (`include/tm_cuda.h`).  The library is built
//! by nvcc, not by cargo: `python -m tuckmill_b200.build` (or the equivalent
//! `nvcc -gencode arch=compute_100a,code=sm_100a -shared` over
//! `tuckmill_b200/csrc/*.cu`) produces `libtm_cuda.so`; this script only tells
//! rustc where it is.  `TM_CUDA_LIB_DIR` names the directory; without it the
//! crate still compiles and every entry point reports `Unavailable` at run
//! time (the same behaviour the Metal crate has off macOS: a forced
//! `--kernels cuda` is refused with a typed error, never a silent fallback).

fn main() {
    println!("cargo:rerun-if-env-changed=TM_CUDA_LIB_DIR");
    println!("cargo:rerun-if-changed=../../include/tm_cuda.h");
    println!("cargo:rustc-check-cfg=cfg(tm_cuda_linked)");
    if let Ok(dir) = std::env::var("TM_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-lib=dylib=tm_cuda");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
        println!("cargo:rustc-cfg=tm_cuda_linked");
    }
}
