// Points the linker at libw8a8.so.  W8A8_LIB_DIR names the directory that holds it (the library's repository builds it
// into inferrous_b200/lib/ with `python -m inferrous_b200.build`).
fn main() {
    println!("cargo:rerun-if-env-changed=W8A8_LIB_DIR");
    if let Ok(dir) = std::env::var("W8A8_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=w8a8");
}
