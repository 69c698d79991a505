// Links libslha_b200.so.  SLHA_B200_LIB_DIR names the directory that holds it
// (the repository builds it in slhav2_b200/); the library itself links only the
// CUDA runtime and binds NCCL at run time.
fn main() {
    println!("cargo:rerun-if-env-changed=SLHA_B200_LIB_DIR");
    if let Ok(dir) = std::env::var("SLHA_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=slha_b200");
}
