// build.rs - compile the CUDA sources for sm_100a and link the shared library.
// Expects this repository's `paged_infer_b200/csrc` and `include` next to the crate (adjust CUDA_SRC / CUDA_INC).
// Not compiled in this repository's environment (no cargo / rustc): shipped as source.
fn main() {
    let out = std::path::PathBuf::from(std::env::var("OUT_DIR").unwrap());
    let src_dir = std::env::var("PAGED_INFER_CUDA_SRC").unwrap_or_else(|_| "../../paged_infer_b200/csrc".into());
    let inc_dir = std::env::var("PAGED_INFER_CUDA_INC").unwrap_or_else(|_| "../../include".into());
    let srcs = ["pi_api", "pi_attention", "pi_attention_flat", "pi_attention_prefill", "pi_attention_prefill_tc", "pi_gemm_tc", "pi_gemv", "pi_glue", "pi_model", "pi_tp"];
    let mut objs = vec![];
    for s in srcs {
        let o = out.join(format!("{s}.o"));
        let st = std::process::Command::new("nvcc")
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", &inc_dir, "-c"])
            .arg(format!("{src_dir}/{s}.cu"))
            .arg("-o")
            .arg(&o)
            .status()
            .expect("nvcc not found");
        assert!(st.success(), "nvcc failed on {s}.cu");
        println!("cargo:rerun-if-changed={src_dir}/{s}.cu");
        objs.push(o);
    }
    let lib = out.join("libpaged_infer_cuda.so");
    let st = std::process::Command::new("nvcc").arg("-shared").arg("-o").arg(&lib).args(&objs).arg("-ldl").status().unwrap();
    assert!(st.success(), "link failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=paged_infer_cuda");
}
