// Tells rustc where libvearo_b200.so lives: VEARO_B200_LIB_DIR, or ../vearo_b200 beside this crate.
fn main() {
    let dir = std::env::var("VEARO_B200_LIB_DIR").unwrap_or_else(|_| {
        let here = std::env::var("CARGO_MANIFEST_DIR").unwrap();
        format!("{here}/../vearo_b200")
    });
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=vearo_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    println!("cargo:rerun-if-env-changed=VEARO_B200_LIB_DIR");
}
