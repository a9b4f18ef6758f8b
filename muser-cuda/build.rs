// Links libmuser_cuda.so (built by `python -m muser_b200.build`).  MUSER_CUDA_LIB_DIR names the folder that holds it.
fn main() {
    println!("cargo:rerun-if-env-changed=MUSER_CUDA_LIB_DIR");
    if let Ok(dir) = std::env::var("MUSER_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=muser_cuda");
}
