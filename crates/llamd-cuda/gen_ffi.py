#!/usr/bin/env python
"""Write crates/llamd-cuda/src/ffi.rs from include/*.h.

Every function the three headers declare becomes one line of an `unsafe extern "C"` block, with the C types mapped
one to one (int -> c_int, const float * -> *const f32, ...). The safe wrappers in lib.rs / forward.rs / batch.rs /
model.rs are written by hand; this file only keeps the raw boundary in step with the headers.

    python crates/llamd-cuda/gen_ffi.py            # rewrite src/ffi.rs
    python crates/llamd-cuda/gen_ffi.py --check    # exit 1 if src/ffi.rs is out of date
"""
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
HEADERS = ["llamd_cuda.h", "llamd_cuda_model.h", "llamd_gguf.h"]

SCALARS = {
    "void": "c_void", "char": "c_char", "int": "c_int", "unsigned int": "c_uint", "long long": "c_longlong",
    "unsigned long long": "c_ulonglong", "size_t": "usize", "float": "f32", "double": "f64",
    "int8_t": "i8", "uint8_t": "u8", "int16_t": "i16", "uint16_t": "u16", "int32_t": "i32", "uint32_t": "u32",
    "int64_t": "i64", "uint64_t": "u64",
    "llamd_model": "llamd_model", "llamd_gguf": "llamd_gguf", "llamd_hparams": "llamd_hparams",
}
RUST_KEYWORDS = {"type", "ref", "in", "box", "move", "fn", "mod", "use", "where", "match", "loop", "as", "impl", "self", "super"}


def strip(text):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    return re.sub(r"^\s*#[^\n]*", "", text, flags=re.M)


def declarations(header):
    """-> [(name, return C type, [(C type, name)])] in header order."""
    text = strip(open(os.path.join(ROOT, "include", header)).read())
    out = []
    for m in re.finditer(r"([A-Za-z_][A-Za-z0-9_ \*]*?)\b(llamd_(?:cuda|fwd|model|gguf)_\w+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.S):
        ret, name, args = re.sub(r"\s+", " ", m.group(1)).strip(), m.group(2), re.sub(r"\s+", " ", m.group(3)).strip()
        params = []
        if args and args != "void":
            for a in args.split(","):
                a = re.sub(r"^(.*?)(\w+)\s*\[\d*\]$", r"\1*\2", a.strip())  # an array parameter is a pointer
                mm = re.match(r"^(.*?)(\w+)$", a)
                params.append((mm.group(1).strip(), mm.group(2)))
        out.append((name, ret, params))
    return out


def rust_type(c):
    """A C type as written in the headers -> the Rust FFI type."""
    c = re.sub(r"\s+", " ", c.replace("*", " * ")).strip()
    toks = c.split(" ")
    # base: everything up to the first '*', minus const/struct
    base, rest, base_const = [], [], False
    i = 0
    while i < len(toks) and toks[i] != "*":
        if toks[i] == "const":
            base_const = True
        elif toks[i] != "struct":
            base.append(toks[i])
        i += 1
    rest = toks[i:]
    ty = SCALARS[" ".join(base)]
    is_const = base_const
    for t in rest:  # each '*' makes a pointer to what is on its left; a following 'const' qualifies that pointer
        if t == "*":
            ty = ("*const " if is_const else "*mut ") + ty
            is_const = False
        elif t == "const":
            is_const = True
    return ty


def render():
    lines = [
        "//! The raw boundary of the CUDA library: one declaration per function of include/llamd_cuda.h,",
        "//! include/llamd_cuda_model.h and include/llamd_gguf.h. WRITTEN BY gen_ffi.py -- edit the headers, then rerun it.",
        "//! Nothing here checks anything; the safe wrappers of this crate validate lengths and ids before they call in.",
        "#![allow(non_camel_case_types, dead_code, clippy::too_many_arguments)]",
        "",
        "use std::os::raw::{c_char, c_int, c_longlong, c_uint, c_ulonglong, c_void};",
        "",
        "/// Opaque handles of the library.",
        "#[repr(C)]",
        "pub struct llamd_model {",
        "    _private: [u8; 0],",
        "}",
        "#[repr(C)]",
        "pub struct llamd_gguf {",
        "    _private: [u8; 0],",
        "}",
        "",
        "/// `llamd_hparams` of include/llamd_cuda_model.h, field for field.",
        "#[repr(C)]",
        "#[derive(Debug, Clone, Copy, Default, PartialEq)]",
        "pub struct llamd_hparams {",
    ]
    text = strip(open(os.path.join(ROOT, "include", "llamd_cuda_model.h")).read())
    body = re.search(r"typedef struct(?: \w+)? \{(.*?)\} llamd_hparams;", text, flags=re.S).group(1)
    for decl in body.split(";"):
        decl = re.sub(r"\s+", " ", decl).strip()
        if not decl:
            continue
        ty, names = decl.split(" ", 1)
        for n in names.split(","):
            lines.append(f"    pub {n.strip()}: {SCALARS[ty]},")
    lines += ["}", ""]
    for h in HEADERS:
        lines.append(f"// ---- include/{h}")
        lines.append('unsafe extern "C" {')
        for name, ret, params in declarations(h):
            ps = ", ".join(f"{(p + '_') if p in RUST_KEYWORDS else p}: {rust_type(t)}" for t, p in params)
            r = "" if ret == "void" else f" -> {rust_type(ret)}"
            lines.append(f"    pub fn {name}({ps}){r};")
        lines += ["}", ""]
    return "\n".join(lines)


def main():
    path = os.path.join(HERE, "src", "ffi.rs")
    text = render()
    if "--check" in sys.argv:
        ok = os.path.exists(path) and open(path).read() == text
        print("ffi.rs is up to date" if ok else "ffi.rs is OUT OF DATE: run python crates/llamd-cuda/gen_ffi.py")
        sys.exit(0 if ok else 1)
    open(path, "w").write(text)
    print(f"wrote {path}: {sum(len(declarations(h)) for h in HEADERS)} functions")


if __name__ == "__main__":
    main()
