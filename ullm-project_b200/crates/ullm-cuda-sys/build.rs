//! Builds `libullm_cuda.so` (hand-written CUDA for sm_100a, nothing else) and checks that the struct
//! layouts declared in `src/lib.rs` are the ones the C header produces.
//!
//! NOT COMPILED in the environment this file was written in (no Rust toolchain there).
//!
//! Counterpart of `crates/ullm-hip-sys/build.rs` in the reference: that script drives CMake, optionally the
//! ROCm compiler, and compares a layout probe's output with the checked-in bindings (`build.rs:330-408`).
//! Here the native build is a plain Makefile (nvcc), and the layout check compiles a ten-line C program.

use std::env;
use std::fs;
use std::path::PathBuf;
use std::process::Command;

/// (C type, size, [(field, offset)]) as declared in src/lib.rs; the probe prints the same from the header.
const LAYOUTS: &[(&str, usize, &[(&str, usize)])] = &[
    ("ullm_cuda_error_sink_t", 48, &[("message", 8), ("message_capacity", 16), ("message_length", 24), ("reserved", 32)]),
    ("ullm_cuda_version_info_t", 32, &[("major", 8), ("reserved", 20)]),
    ("ullm_cuda_backend_probe_result_t", 64, &[("backend", 8), ("global_memory_bytes", 40), ("reserved", 48)]),
    ("ullm_cuda_context_probe_result_t", 32, &[("context_present", 8), ("reserved", 20)]),
    ("ullm_cuda_tensor_t", 16, &[("buffer", 0), ("offset_bytes", 8)]),
    ("ullm_cuda_weight_t", 56, &[("n", 8), ("k", 16), ("values", 24), ("scales", 40)]),
    ("ullm_cuda_completion_result_t", 56, &[("dispatch_count", 8), ("selected_backend", 24), ("device_flags", 36)]),
    ("ullm_cuda_linear_desc_t", 200, &[("weight", 8), ("m", 64), ("input", 72), ("output", 96), ("input_dtype", 120),
                                        ("norm_weight", 144), ("residual", 160), ("residual_row_stride", 176), ("reserved", 184)]),
    ("ullm_cuda_slots_t", 64, &[("slots", 8), ("rank_stride_bytes", 24), ("ranks", 32), ("reserved", 48)]),
    ("ullm_cuda_stack_desc_t", 88, &[("encoding", 8), ("seed", 56), ("rms_eps", 64)]),
    ("ullm_cuda_stack_linear_info_t", 208, &[("weight", 8), ("last_input", 104), ("last_output", 120), ("norm_weight", 152),
                                              ("last_residual", 168), ("norm_tensor_id", 184)]),
];

fn run(cmd: &mut Command, what: &str) -> String {
    let out = cmd.output().unwrap_or_else(|e| panic!("failed to start {what}: {e}"));
    assert!(out.status.success(), "{what} failed: {}\n{}", out.status, String::from_utf8_lossy(&out.stderr));
    String::from_utf8_lossy(&out.stdout).into_owned()
}

fn main() {
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap());
    // crates/ullm-cuda-sys -> repository root that holds include/ullm_cuda.h and the CUDA sources
    let root = env::var("ULLM_CUDA_SOURCE_ROOT").map(PathBuf::from).unwrap_or_else(|_| manifest.join("../../.."));
    let header_dir = root.join("include");
    let csrc = root.join("ullm-project_b200/csrc");
    let out_dir = PathBuf::from(env::var("OUT_DIR").unwrap());
    println!("cargo:rerun-if-changed={}", header_dir.join("ullm_cuda.h").display());
    println!("cargo:rerun-if-changed={}", csrc.display());
    println!("cargo:rerun-if-env-changed=ULLM_CUDA_SOURCE_ROOT");
    println!("cargo:rerun-if-env-changed=NVCC");

    // 1. layout probe: the header's view of every struct this crate mirrors
    let mut src = String::from("#include <stddef.h>\n#include <stdio.h>\n#include \"ullm_cuda.h\"\nint main(void){\n");
    for (ty, _, fields) in LAYOUTS {
        src += &format!("printf(\"{ty} %zu\\n\", sizeof({ty}));\n");
        for (f, _) in *fields {
            src += &format!("printf(\"{ty}.{f} %zu\\n\", offsetof({ty}, {f}));\n");
        }
    }
    src += "return 0;}\n";
    let probe_c = out_dir.join("layout_probe.c");
    let probe = out_dir.join("layout_probe");
    fs::write(&probe_c, src).unwrap();
    let cc = env::var("CC").unwrap_or_else(|_| "cc".into());
    run(Command::new(&cc).arg("-std=c99").arg("-I").arg(&header_dir).arg(&probe_c).arg("-o").arg(&probe), "layout probe build");
    let seen = run(&mut Command::new(&probe), "layout probe");
    for (ty, size, fields) in LAYOUTS {
        assert!(seen.contains(&format!("{ty} {size}\n")), "size of {ty} differs from src/lib.rs: header says\n{seen}");
        for (f, off) in *fields {
            assert!(seen.contains(&format!("{ty}.{f} {off}\n")), "offset of {ty}.{f} differs from src/lib.rs");
        }
    }

    // 2. the native library: sm_100a only, no other target and no CPU code path
    let mut make = Command::new("make");
    make.arg("-C").arg(&csrc).arg("-j8");
    if let Ok(nvcc) = env::var("NVCC") {
        make.arg(format!("NVCC={nvcc}"));
    }
    run(&mut make, "libullm_cuda build (nvcc, sm_100a)");
    let lib_dir = root.join("ullm-project_b200/lib");
    println!("cargo:rustc-link-search=native={}", lib_dir.display());
    println!("cargo:rustc-link-lib=dylib=ullm_cuda");
    println!("cargo:lib_dir={}", lib_dir.display());
}
