// NOT COMPILED IN THIS ENVIRONMENT.
//
// Builds libcandle_b200.so (and, with the `nccl` feature, libcandle_b200_nccl.so) with nvcc for
// sm_100a and tells cargo to link them.  Modelled on candle-flash-attn/build.rs:73-102, which drives
// nvcc through bindgen_cuda; here the sources are few enough to call nvcc directly.
//
//   CANDLE_B200_SRC        directory holding candle_b200/csrc and include/ (default: ../../ relative to
//                          this crate, i.e. the repository this crate ships in)
//   CANDLE_B200_BUILD_DIR  where the libraries go (default: OUT_DIR), like CANDLE_FLASH_ATTN_BUILD_DIR
//   CANDLE_B200_PREBUILT   if set, skip nvcc and link the libraries found in this directory
use std::path::PathBuf;
use std::process::Command;

// every .cu of candle_b200/csrc goes into the core library except this one (the NCCL entry points)
const NCCL_SOURCE: &str = "sharded.cu";

fn main() -> anyhow::Result<()> {
    println!("cargo:rerun-if-changed=build.rs");
    for var in ["CANDLE_B200_SRC", "CANDLE_B200_BUILD_DIR", "CANDLE_B200_PREBUILT"] {
        println!("cargo:rerun-if-env-changed={var}");
    }
    let out_dir = PathBuf::from(std::env::var("OUT_DIR")?);
    if let Ok(dir) = std::env::var("CANDLE_B200_PREBUILT") {
        link(&PathBuf::from(dir));
        return Ok(());
    }
    let src = match std::env::var("CANDLE_B200_SRC") {
        Ok(s) => PathBuf::from(s),
        Err(_) => PathBuf::from(std::env::var("CARGO_MANIFEST_DIR")?).join("../.."),
    };
    let csrc = src.join("candle_b200/csrc");
    let build_dir = match std::env::var("CANDLE_B200_BUILD_DIR") {
        Ok(d) => PathBuf::from(d),
        Err(_) => out_dir,
    };
    std::fs::create_dir_all(&build_dir)?;
    let nvcc = std::env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());
    let common = [
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared",
    ];
    let core = build_dir.join("libcandle_b200.so");
    let mut cmd = Command::new(&nvcc);
    cmd.args(common).arg("-o").arg(&core);
    for entry in std::fs::read_dir(&csrc)? {
        let p = entry?.path();
        println!("cargo:rerun-if-changed={}", p.display());
        let is_cu = p.extension().map(|e| e == "cu").unwrap_or(false);
        if is_cu && p.file_name().map(|n| n != NCCL_SOURCE).unwrap_or(false) {
            cmd.arg(p);
        }
    }
    anyhow::ensure!(cmd.status()?.success(), "nvcc failed for libcandle_b200.so");
    if cfg!(feature = "nccl") {
        let status = Command::new(&nvcc)
            .args(common)
            .arg("-o")
            .arg(build_dir.join("libcandle_b200_nccl.so"))
            .arg(csrc.join(NCCL_SOURCE))
            .arg(format!("-L{}", build_dir.display()))
            .args(["-l:libcandle_b200.so", "-Xlinker", "-rpath=$ORIGIN", "-lnccl"])
            .status()?;
        anyhow::ensure!(status.success(), "nvcc failed for libcandle_b200_nccl.so");
    }
    link(&build_dir);
    Ok(())
}

fn link(dir: &PathBuf) {
    println!("cargo:rustc-link-search={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=candle_b200");
    if cfg!(feature = "nccl") {
        println!("cargo:rustc-link-lib=dylib=candle_b200_nccl");
    }
    println!("cargo:rustc-link-lib=dylib=cudart");
    println!("cargo:rustc-link-lib=dylib=stdc++");
}
