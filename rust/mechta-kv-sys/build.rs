// Points the linker at libmechta_kv.so. MECHTA_KV_LIB_DIR names the directory that holds it (the `mechta_b200`
// directory of the library's tree after `make -C mechta_b200/csrc`).
fn main() {
    if let Ok(dir) = std::env::var("MECHTA_KV_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=mechta_kv");
    println!("cargo:rerun-if-env-changed=MECHTA_KV_LIB_DIR");
}
