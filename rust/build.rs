// build.rs: compiles libsgk.so (the CUDA kernels and their C ABI) with nvcc for sm_100a and
// links the crate against it. Takes the place of the reference's build.rs, which only copies
// the frozen Metal preamble into OUT_DIR (build.rs:3-11 of the reference).
//
// SGK_ROOT names the checkout that holds saragossa_b200/csrc and include/sgk.h; NVCC overrides
// the compiler. There is no CPU fallback: without nvcc the build fails.
//
// Not compiled where this repository is built (no Rust toolchain there); the same nvcc line
// is what saragossa_b200/build.py runs and what the tests load.
use std::path::PathBuf;
use std::process::Command;

fn main() {
    let root = PathBuf::from(std::env::var("SGK_ROOT").expect("SGK_ROOT: path of the saragossa_b200 checkout"));
    let csrc = root.join("saragossa_b200").join("csrc");
    let out = PathBuf::from(std::env::var("OUT_DIR").expect("OUT_DIR"));
    let nvcc = std::env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());

    let mut sources: Vec<PathBuf> = std::fs::read_dir(&csrc)
        .expect("saragossa_b200/csrc")
        .filter_map(|e| e.ok().map(|e| e.path()))
        .filter(|p| p.extension().map(|x| x == "cu").unwrap_or(false))
        .collect();
    sources.sort();
    assert!(!sources.is_empty(), "no .cu sources under {}", csrc.display());

    let lib = out.join("libsgk.so");
    let mut cmd = Command::new(&nvcc);
    cmd.args([
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
        "-Xcompiler", "-fPIC", "-shared", "-cudart", "static", "-o",
    ])
    .arg(&lib);
    for s in &sources {
        cmd.arg(s);
        println!("cargo:rerun-if-changed={}", s.display());
    }
    for h in ["host.h", "kernels.h", "layout.h", "device_common.cuh", "mma_common.cuh"] {
        println!("cargo:rerun-if-changed={}", csrc.join(h).display());
    }
    println!("cargo:rerun-if-changed={}", root.join("include").join("sgk.h").display());
    println!("cargo:rerun-if-env-changed=SGK_ROOT");
    println!("cargo:rerun-if-env-changed=NVCC");
    let status = cmd.status().unwrap_or_else(|e| panic!("could not run {nvcc}: {e}"));
    assert!(status.success(), "nvcc failed building {}", lib.display());

    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=sgk");
    // the runtime loader must find the library next to the crate's artefacts
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", out.display());
}
