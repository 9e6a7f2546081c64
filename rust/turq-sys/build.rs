// Links the prebuilt libturq.so. TURQ_LIB_DIR names the directory that holds it (the
// `tur_b200/` folder of the repository after `python -m tur_b200.build`); the CUDA runtime it
// depends on is found through the usual loader path.
use std::env;

fn main() {
    println!("cargo:rerun-if-env-changed=TURQ_LIB_DIR");
    if let Ok(dir) = env::var("TURQ_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=turq");
}
