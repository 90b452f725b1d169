// COMPILE-UNVERIFIED (no Rust toolchain where this was written).
//
// Links the prebuilt C-ABI library.  WETA_B200_LIB_DIR names the directory that holds libweta_b200.so
// (built by `make -C weta_b200/csrc` in the weta_b200 repository: nvcc, sm_100a, no run-time compilation).
use std::env;

fn main() {
    println!("cargo:rerun-if-env-changed=WETA_B200_LIB_DIR");
    let dir = env::var("WETA_B200_LIB_DIR").unwrap_or_else(|_| "/usr/local/lib".to_string());
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=weta_b200");
    // so that the test binaries find it without LD_LIBRARY_PATH
    println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
}
