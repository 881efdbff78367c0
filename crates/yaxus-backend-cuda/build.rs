// UNVERIFIED: no rustc in the image this repository is built in; never compiled.
//
// Compiles the CUDA sources of libyaxus_cuda for sm_100a and links the crate against the
// result.  YAXUS_CUDA_SRC names the directory that holds the sources (`yaxus_b200/csrc` of the
// library's repository) and YAXUS_CUDA_INCLUDE the one with `yaxus_cuda.h`; by default both are
// looked for under `vendor/` of this crate.  The same commands, for Python users, are in
// `yaxus_b200/build.py` of the library.
use std::{env, path::PathBuf, process::Command};

const SOURCES: &[&str] = &[
    "api.cu", "kv_ops.cu", "attend_simt.cu", "attend_mma.cu", "prefill_tc.cu", "combine.cu", "dist.cu",
    "attend_static.cu", "planner.cpp", "hooks.cu",
];

fn main() {
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let here = PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap());
    let src = env::var("YAXUS_CUDA_SRC").map(PathBuf::from).unwrap_or_else(|_| here.join("vendor/csrc"));
    println!("cargo:rerun-if-env-changed=YAXUS_CUDA_SRC");
    println!("cargo:rerun-if-changed={}", src.display());
    let mut objects = Vec::new();
    for s in SOURCES {
        let obj = out.join(format!("{s}.o"));
        let ok = Command::new("nvcc")
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17"])
            .args(["-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-x", "cu", "-c"])
            .arg(src.join(s))
            .arg("-o")
            .arg(&obj)
            .status()
            .expect("nvcc not found: the CUDA toolkit (12.8 or later, for sm_100a) must be installed")
            .success();
        assert!(ok, "nvcc failed on {s}");
        objects.push(obj);
    }
    let lib = out.join("libyaxus_cuda.so");
    let ok = Command::new("nvcc").arg("-shared").arg("-o").arg(&lib).args(&objects).arg("-ldl").status().unwrap().success();
    assert!(ok, "linking libyaxus_cuda.so failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=yaxus_cuda");
}
