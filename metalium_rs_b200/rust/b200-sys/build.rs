// Builds libb200tt from metalium_rs_b200/csrc with nvcc for sm_100a and links it statically.
// `python -m metalium_rs_b200.build` runs the same nvcc command lines where there is no cargo.
fn main() {
    let out = std::path::PathBuf::from(std::env::var("OUT_DIR").unwrap());
    let csrc = std::path::Path::new("../../csrc");
    let units = [("engine.cu", false), ("k_eltwise.cu", true), ("k_reduce.cu", true), ("k_index.cu", false),
                 ("k_gemm_simt.cu", false), ("k_gemm_tc.cu", false), ("k_gemm_tc2.cu", false), ("k_gemm_addnorm.cu", true), ("k_gemm_tf32.cu", false),
                 ("k_gemm_skinny.cu", false), ("k_attention.cu", false), ("k_attention_tc.cu", false),
                 ("k_convert.cu", false), ("k_bfp.cu", false), ("k_decode.cu", false), ("k_pool.cu", true), ("k_scan_sort.cu", true), ("k_random.cu", true)];
    let mut objs = vec![];
    for (src, separate_roundings) in units {
        let obj = out.join(src.replace(".cu", ".o"));
        let mut c = std::process::Command::new("nvcc");
        c.args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]);
        if separate_roundings { c.arg("-fmad=false"); }  // kinds the reference defines as separate roundings
        c.arg("-c").arg(csrc.join(src)).arg("-o").arg(&obj);
        assert!(c.status().expect("nvcc").success(), "nvcc failed on {src}");
        println!("cargo:rerun-if-changed={}", csrc.join(src).display());
        objs.push(obj);
    }
    let lib = out.join("libb200tt.a");
    assert!(std::process::Command::new("ar").arg("crs").arg(&lib).args(&objs).status().unwrap().success());
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-search=native=/usr/local/cuda/lib64");
    println!("cargo:rustc-link-lib=static=b200tt");
    println!("cargo:rustc-link-lib=static=cudart_static");
    println!("cargo:rustc-link-lib=dylib=stdc++");
    println!("cargo:rustc-link-lib=dylib=dl");
    println!("cargo:rustc-link-lib=dylib=rt");
}
