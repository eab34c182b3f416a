// Links libllmini_b200.so (built by `python -m llmini_b200.build`); LLMINI_B200_LIB_DIR names its folder.
fn main() {
    let dir = std::env::var("LLMINI_B200_LIB_DIR").expect("set LLMINI_B200_LIB_DIR to llmini_b200/_lib");
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=llmini_b200");
    println!("cargo:rerun-if-env-changed=LLMINI_B200_LIB_DIR");
}
