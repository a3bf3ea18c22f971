// NOT COMPILED IN THE BUILD ENVIRONMENT OF THIS REPOSITORY (no cargo / rustc).
//
// Resolves the prebuilt libhs_attn.so the way crates/bitsandbytes-sys/build.rs:86-163 resolves libbitsandbytes:
// an environment variable first, then a few conventional directories; emits the link directives, links the CUDA
// runtime's dependencies and sets cfg(hs_attn_cuda) so that the caller can compile the feature out when the library is
// absent.  The library itself is built by `python hyprstream_b200/csrc/build.py` (nvcc, sm_100a).
use std::env;
use std::path::PathBuf;

fn find_library() -> Option<PathBuf> {
    // 1. HS_ATTN_LIB_DIR=/path/to/dir/containing/libhs_attn.so   (or HS_ATTN_LIB_PATH=/path/to/libhs_attn.so)
    if let Ok(p) = env::var("HS_ATTN_LIB_PATH") {
        let p = PathBuf::from(p);
        if p.is_file() {
            return p.parent().map(|d| d.to_path_buf());
        }
    }
    let mut dirs: Vec<PathBuf> = Vec::new();
    if let Ok(d) = env::var("HS_ATTN_LIB_DIR") {
        dirs.push(PathBuf::from(d));
    }
    // 2. beside this crate, where the repository's build script puts it
    if let Ok(manifest) = env::var("CARGO_MANIFEST_DIR") {
        dirs.push(PathBuf::from(&manifest).join("../../hyprstream_b200"));
    }
    // 3. system directories
    for d in ["/usr/local/lib", "/usr/lib", "/usr/lib64"] {
        dirs.push(PathBuf::from(d));
    }
    dirs.into_iter().find(|d| d.join("libhs_attn.so").is_file())
}

fn main() {
    println!("cargo:rerun-if-env-changed=HS_ATTN_LIB_DIR");
    println!("cargo:rerun-if-env-changed=HS_ATTN_LIB_PATH");
    println!("cargo:rustc-check-cfg=cfg(hs_attn_cuda)");
    match find_library() {
        Some(dir) => {
            println!("cargo:rustc-link-search=native={}", dir.display());
            println!("cargo:rustc-link-lib=dylib=hs_attn");
            // libhs_attn links the CUDA runtime statically; what remains are its system dependencies
            for lib in ["dl", "pthread", "rt", "stdc++"] {
                println!("cargo:rustc-link-lib=dylib={}", lib);
            }
            println!("cargo:rustc-cfg=hs_attn_cuda");
            println!("cargo:lib_dir={}", dir.display());
        }
        None => {
            if env::var("CARGO_FEATURE_REQUIRE_LIB").is_ok() {
                panic!("libhs_attn.so not found: set HS_ATTN_LIB_DIR, or build it with `python hyprstream_b200/csrc/build.py`");
            }
            println!("cargo:warning=libhs_attn.so not found; hyprstream-attn-sys is compiled without cfg(hs_attn_cuda)");
        }
    }
}
