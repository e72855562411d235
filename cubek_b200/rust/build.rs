// Links against libcubek_quant_b200.so; set CUBEK_QUANT_B200_LIB_DIR to the directory that holds it.
fn main() {
    if let Ok(dir) = std::env::var("CUBEK_QUANT_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=cubek_quant_b200");
    println!("cargo:rerun-if-env-changed=CUBEK_QUANT_B200_LIB_DIR");
}
