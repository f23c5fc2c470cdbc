// Links libzkb200.so. ZKB200_LIB_DIR is the directory `python -m zk_inference_prover_b200.build` wrote the library to
// (zk_inference_prover_b200/lib); the CUDA runtime is linked statically into it, so nothing else is needed.
fn main() {
    let dir = std::env::var("ZKB200_LIB_DIR").expect("set ZKB200_LIB_DIR to the directory that holds libzkb200.so");
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=zkb200");
    println!("cargo:rerun-if-env-changed=ZKB200_LIB_DIR");
}
