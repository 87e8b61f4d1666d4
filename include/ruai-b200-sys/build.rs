// Locates libruai_b200.so.  RUAI_B200_LIB_DIR names the directory that holds it (the `ruai_b200/`
// package directory of the library's tree after `python -m ruai_b200._build`); the default is that
// directory relative to this crate.  The library itself is built by nvcc for sm_100a, not by cargo.
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("RUAI_B200_LIB_DIR")
        .map(PathBuf::from)
        .unwrap_or_else(|_| PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../ruai_b200"));
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=ruai_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
    println!("cargo:rerun-if-env-changed=RUAI_B200_LIB_DIR");
    println!("cargo:rerun-if-changed=../ruai_b200.h");
}
