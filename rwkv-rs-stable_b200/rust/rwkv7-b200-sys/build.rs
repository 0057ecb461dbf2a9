//! Builds `librwkv7_b200.so` with the repository's own build script and tells cargo where it is.
//!
//! `RWKV7_B200_LIB_DIR` points at a directory that already holds the library (a packaged build);
//! otherwise `python <root>/rwkv-rs-stable_b200/build.py` is run, which calls
//! `nvcc -gencode arch=compute_100a,code=sm_100a` on the sources under `csrc/` and leaves the
//! library in the package directory.
use std::env;
use std::path::PathBuf;
use std::process::Command;

fn main() {
    println!("cargo:rerun-if-env-changed=RWKV7_B200_LIB_DIR");
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").expect("cargo sets CARGO_MANIFEST_DIR"));
    // <package>/rust/rwkv7-b200-sys  ->  <package>
    let package = manifest.parent().and_then(|p| p.parent()).expect("crate sits two levels below the package").to_path_buf();
    let lib_dir = match env::var("RWKV7_B200_LIB_DIR") {
        Ok(dir) => PathBuf::from(dir),
        Err(_) => {
            let script = package.join("build.py");
            println!("cargo:rerun-if-changed={}", package.join("csrc").display());
            let status = Command::new("python").arg(&script).status().expect("python is needed to run build.py");
            assert!(status.success(), "{} failed", script.display());
            package.clone()
        }
    };
    assert!(lib_dir.join("librwkv7_b200.so").exists(), "librwkv7_b200.so not found in {}", lib_dir.display());
    println!("cargo:rustc-link-search=native={}", lib_dir.display());
    println!("cargo:rustc-link-lib=dylib=rwkv7_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", lib_dir.display());
    // for dependants that want the C header (bindgen users)
    println!("cargo:include={}", package.parent().expect("package has a parent").join("include").display());
}
