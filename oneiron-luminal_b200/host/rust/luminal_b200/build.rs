// Links the prebuilt C-ABI library.  LUM_B200_LIB_DIR points at the directory that holds liblum_b200.so
// (by default the package directory of this repository: three levels up from the crate).
use std::{env, path::PathBuf};

fn main() {
    let dir = env::var("LUM_B200_LIB_DIR")
        .map(PathBuf::from)
        .unwrap_or_else(|_| PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../.."));
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=lum_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
    println!("cargo:rerun-if-env-changed=LUM_B200_LIB_DIR");
}
