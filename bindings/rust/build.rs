// Links against libnixl_capi.so of an in-tree build.  NIXL_B200_LIB_DIR names the directory that
// holds it (default: ../../nixl_b200/lib relative to this crate).
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("NIXL_B200_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../nixl_b200/lib")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=nixl_capi");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
    println!("cargo:rerun-if-env-changed=NIXL_B200_LIB_DIR");
}
