// Points rustc at libhearth_b200.so.  HEARTH_B200_LIB_DIR names the directory that holds it (the
// hearth_b200/ folder of the CUDA build); without it the default linker search path is used.
fn main() {
    println!("cargo:rerun-if-env-changed=HEARTH_B200_LIB_DIR");
    if let Ok(dir) = std::env::var("HEARTH_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={}", dir);
        println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir);
    }
    println!("cargo:rustc-link-lib=dylib=hearth_b200");
}
