// Links libetcuda.so from ETCUDA_LIB_DIR (the directory that holds the library built from effect_torch_b200/csrc) and,
// for the addon build, runs the napi set-up.
fn main() {
    if let Ok(dir) = std::env::var("ETCUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=etcuda");
    println!("cargo:rerun-if-env-changed=ETCUDA_LIB_DIR");
    #[cfg(feature = "napi")]
    napi_build::setup();
}
