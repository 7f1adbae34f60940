// Builds libtangq.so with nvcc (sm_100a only) from the CUDA sources of this repository and tells cargo to link it.
// The same command as tang_b200/_build.py; TANGQ_LIB_DIR skips the build and links an existing library.
use std::env;
use std::path::PathBuf;
use std::process::Command;

fn main() {
    println!("cargo:rerun-if-env-changed=TANGQ_LIB_DIR");
    if let Ok(dir) = env::var("TANGQ_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-lib=dylib=tangq");
        return;
    }
    let root = PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../..");
    let csrc = root.join("tang_b200/csrc");
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let lib = out.join("libtangq.so");
    let mut sources = Vec::new();
    for entry in std::fs::read_dir(&csrc).expect("tang_b200/csrc") {
        let path = entry.unwrap().path();
        println!("cargo:rerun-if-changed={}", path.display());
        if path.extension().map(|e| e == "cu").unwrap_or(false) {
            sources.push(path);
        }
    }
    sources.sort();
    println!("cargo:rerun-if-changed={}", root.join("include/tangq.h").display());
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());
    let status = Command::new(nvcc)
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17"])
        .args(["-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared", "-ldl", "-o"])
        .arg(&lib)
        .args(&sources)
        .status()
        .expect("nvcc not found (set NVCC or TANGQ_LIB_DIR)");
    assert!(status.success(), "nvcc failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=tangq");
    println!("cargo:rustc-link-lib=dylib=cudart");
}
