"""The Rust crate sources (crates/llamd-cuda, crates/llamd-runtime/src/cuda_model.rs) against the C headers.

There is no Rust toolchain where these sources were written, so they cannot be compiled here. What can be checked
without one is checked:
  - src/ffi.rs is what gen_ffi.py produces from include/*.h today;
  - independently of that generator: every function a header declares appears in ffi.rs with the same number of
    arguments and, argument by argument and for the return value, the Rust type that the C type maps to;
  - every `ffi::` call in the hand-written wrappers names a declared function and passes as many arguments as it takes;
  - every source file has balanced brackets, and the additive `backend.rs` change is present.
"""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CRATE = os.path.join(ROOT, "crates", "llamd-cuda")
HEADERS = ["llamd_cuda.h", "llamd_cuda_model.h", "llamd_gguf.h"]
RUST_FILES = [os.path.join(CRATE, "build.rs")] + [os.path.join(CRATE, "src", f) for f in ("lib.rs", "ffi.rs", "forward.rs", "batch.rs", "model.rs")] + \
             [os.path.join(ROOT, "crates", "llamd-runtime", "src", "cuda_model.rs")]

# C type (normalised: single spaces, '*' attached as ' *') -> Rust type; written out by hand, not shared with gen_ffi.py
C_TO_RUST = {
    "void": None, "int": "c_int", "int32_t": "i32", "uint32_t": "u32", "uint64_t": "u64", "int64_t": "i64", "size_t": "usize",
    "float": "f32", "long long": "c_longlong", "unsigned long long": "c_ulonglong",
    "void *": "*mut c_void", "const void *": "*const c_void", "char *": "*mut c_char", "const char *": "*const c_char",
    "float *": "*mut f32", "const float *": "*const f32", "int8_t *": "*mut i8", "const int8_t *": "*const i8",
    "int16_t *": "*mut i16", "int32_t *": "*mut i32", "const int32_t *": "*const i32", "uint32_t *": "*mut u32",
    "const uint32_t *": "*const u32", "uint64_t *": "*mut u64", "int *": "*mut c_int", "size_t *": "*mut usize",
    "unsigned int *": "*mut c_uint", "llamd_model *": "*mut llamd_model", "llamd_gguf *": "*mut llamd_gguf",
    "const llamd_gguf *": "*const llamd_gguf", "const llamd_hparams *": "*const llamd_hparams", "llamd_hparams *": "*mut llamd_hparams",
    "void **": "*mut *mut c_void", "void *const *": "*const *mut c_void", "const void **": "*mut *const c_void",
    "const char **": "*mut *const c_char", "int32_t": "i32", "uint8_t *": "*mut u8", "const uint8_t *": "*const u8",
    "int64_t *": "*mut i64", "double *": "*mut f64", "unsigned long long *": "*mut c_ulonglong", "long long *": "*mut c_longlong",
}


def strip_c(text):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    return re.sub(r"^\s*#[^\n]*", "", text, flags=re.M)


def norm_c_type(t):
    t = re.sub(r"\s+", " ", t.replace("*", " * ")).strip()
    t = re.sub(r" \* ", " *", t + " ").strip()          # "const float *" ; "void * *" -> "void **"
    t = t.replace("* *", "**").replace("*const *", "*const *")
    return re.sub(r"\s+", " ", t)


def header_functions():
    out = {}
    for h in HEADERS:
        text = strip_c(open(os.path.join(ROOT, "include", h)).read())
        for m in re.finditer(r"([A-Za-z_][A-Za-z0-9_ \*]*?)\b(llamd_(?:cuda|fwd|model|gguf)_\w+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.S):
            ret, name, args = m.group(1), m.group(2), re.sub(r"\s+", " ", m.group(3)).strip()
            params = []
            if args and args != "void":
                for a in args.split(","):
                    a = a.strip()
                    arr = re.match(r"^(.*?)(\w+)\s*\[\d*\]$", a)
                    if arr:
                        params.append(norm_c_type(arr.group(1) + " *"))
                    else:
                        params.append(norm_c_type(re.match(r"^(.*?)(\w+)$", a).group(1)))
            out[name] = (norm_c_type(ret), params)
    return out


def rust_functions():
    text = open(os.path.join(CRATE, "src", "ffi.rs")).read()
    out = {}
    for m in re.finditer(r"pub fn (llamd_\w+)\((.*?)\)( -> ([^;]+))?;", text):
        params = [p.split(":", 1)[1].strip() for p in m.group(2).split(", ")] if m.group(2).strip() else []
        out[m.group(1)] = (m.group(4).strip() if m.group(4) else None, params)
    return out


def test_ffi_rs_is_what_the_generator_writes():
    r = subprocess.run([sys.executable, os.path.join(CRATE, "gen_ffi.py"), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def test_every_header_function_is_declared_with_matching_types():
    c, r = header_functions(), rust_functions()
    assert len(c) > 150
    assert set(c) == set(r), (sorted(set(c) - set(r)), sorted(set(r) - set(c)))
    for name, (ret, params) in c.items():
        rret, rparams = r[name]
        assert C_TO_RUST[ret] == rret, (name, ret, rret)
        assert len(params) == len(rparams), (name, params, rparams)
        for i, (ct, rt) in enumerate(zip(params, rparams)):
            assert ct in C_TO_RUST, (name, i, ct)
            assert C_TO_RUST[ct] == rt, (name, i, ct, rt)


def split_args(s):
    """Top-level comma split of a Rust argument list."""
    args, depth, cur = [], 0, ""
    for ch in s:
        if ch in "([{<" :
            depth += 1
        elif ch in ")]}>":
            depth -= 1
        if ch == "," and depth == 0:
            args.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        args.append(cur)
    return args


def test_wrapper_calls_match_the_declarations():
    decl = rust_functions()
    seen = set()
    for path in RUST_FILES:
        if path.endswith("ffi.rs") or path.endswith("build.rs"):
            continue
        text = re.sub(r"//[^\n]*", "", open(path).read())
        for m in re.finditer(r"ffi::(llamd_\w+)\(", text):
            name = m.group(1)
            assert name in decl, f"{os.path.basename(path)} calls {name}, which no header declares"
            # find the matching parenthesis
            i, depth = m.end(), 1
            while depth:
                depth += {"(": 1, ")": -1}.get(text[i], 0)
                i += 1
            n_args = len(split_args(text[m.end():i - 1].replace("->", "  ")))
            assert n_args == len(decl[name][1]), f"{os.path.basename(path)}: {name} called with {n_args} arguments, declared with {len(decl[name][1])}"
            seen.add(name)
    # the surface the reference's runtime and bench drive is covered
    for must in ("llamd_cuda_device_info", "llamd_cuda_upload_q6k", "llamd_cuda_matvec_q6k_resident", "llamd_cuda_matvec_grouped",
                 "llamd_cuda_quantize_q8k", "llamd_fwd_sync", "llamd_fwd_begin_capture", "llamd_fwd_router", "llamd_fwd_matvec_grouped_x2",
                 "llamd_fwd_matvec_grouped_pa", "llamd_fwd_moe_combine_add", "llamd_fwd_expert_gemm", "llamd_fwd_moe_group",
                 "llamd_model_create", "llamd_model_forward", "llamd_model_forward_batch", "llamd_model_prefill", "llamd_model_decode"):
        assert must in seen, f"no wrapper calls {must}"


def test_sources_are_well_formed_and_say_they_were_not_compiled():
    for path in RUST_FILES:
        text = open(path).read()
        code = re.sub(r'"(?:[^"\\]|\\.)*"', '""', re.sub(r"//[^\n]*", "", text))
        code = re.sub(r"'.'|'\\.'", "' '", code)
        for a, b in ("()", "[]", "{}"):
            assert code.count(a) == code.count(b), f"{os.path.basename(path)}: unbalanced {a}{b}"
    assert "NOT COMPILED" in open(os.path.join(CRATE, "src", "lib.rs")).read()
    assert "NOT COMPILED" in open(os.path.join(CRATE, "build.rs")).read()
    patch = open(os.path.join(ROOT, "crates", "llamd-runtime", "src", "backend_cuda.patch")).read()
    assert "Backend::Cuda => llamd_cuda::available()" in patch and '"cuda" | "nvidia" => Ok(Backend::Cuda)' in patch
    build = open(os.path.join(CRATE, "build.rs")).read()
    assert "compute_100a" in build and "--fmad=false" in build and "cargo::rustc-cfg=cuda" in build
