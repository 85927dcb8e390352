// Links the C-ABI library built from moe4all_b200/csrc (libinfr_cuda.so, sm_100a only).
fn main() {
    println!("cargo:rerun-if-env-changed=INFR_CUDA_LIB_DIR");
    if let Ok(dir) = std::env::var("INFR_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=infr_cuda");
}
