#!/usr/bin/env python
"""Writes rust/ffi.rs from include/sgk.h: one `extern "C"` declaration per prototype of
the header, the opaque handle types, the two plain structs, the status codes and the
status -> InferError mapping the crate's Result surface needs.

    python rust/gen_ffi.py            # rewrites rust/ffi.rs
    python rust/gen_ffi.py --check    # exit 1 when rust/ffi.rs is not what the header gives

The header is the single source of truth; the generated file is committed so that a
maintainer of the crate can drop it in without running Python. No Rust toolchain exists
where this repository is built, so ffi.rs is checked against the header by a test
(tests/test_rust_ffi.py), not by rustc.
"""
from __future__ import annotations

import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(os.path.dirname(HERE), "include", "sgk.h")
OUT = os.path.join(HERE, "ffi.rs")

SCALARS = {
    "int32_t": "i32", "int64_t": "i64", "uint64_t": "u64", "uint32_t": "u32", "uint16_t": "u16",
    "uint8_t": "u8", "size_t": "usize", "float": "f32", "double": "f64", "int": "std::os::raw::c_int",
    "char": "std::os::raw::c_char", "void": "std::ffi::c_void",
}
RUST_KEYWORDS = {"type", "ref", "in", "box", "move", "fn", "mod", "match", "loop", "self", "where"}


def strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def camel(name: str) -> str:
    return "".join(part.capitalize() for part in name.split("_"))


def parse(path: str = HEADER):
    raw = open(path).read()
    text = strip_comments(raw)
    handles = re.findall(r"typedef\s+struct\s+(sgk_\w+)\s+\1\s*;", text)
    structs = []
    for m in re.finditer(r"typedef\s+struct\s*\{(.*?)\}\s*(sgk_\w+)\s*;", text, flags=re.S):
        fields = []
        for decl in m.group(1).split(";"):
            decl = decl.strip()
            if not decl:
                continue
            if "*" in decl:                      # one pointer field per declaration
                name, ctype, _ = parse_param(decl, len(fields))
                fields.append((name, ctype))
                continue
            ctype, names = decl.split(None, 1)
            for name in names.split(","):
                fields.append((name.strip(), ctype))
        structs.append((m.group(2), fields))
    enums = []
    for m in re.finditer(r"enum\s*\{(.*?)\}\s*;", text, flags=re.S):
        for item in m.group(1).split(","):
            item = item.strip()
            if item:
                name, value = [x.strip() for x in item.split("=")]
                enums.append((name, value))
    defines = re.findall(r"^#define\s+(SGK_\w+)\s+(.+?)\s*$", strip_comments(raw), flags=re.M)
    defines = [(n, v) for n, v in defines if n != "SGK_H_"]
    body = re.sub(r"#[^\n]*", " ", text)
    body = re.sub(r"typedef\s+struct\s*\{.*?\}\s*sgk_\w+\s*;", " ", body, flags=re.S)
    protos = []
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(sgk_\w+)\s*\(([^;{}]*?)\)\s*;", body):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if ret.startswith("typedef") or ret.startswith("struct"):
            continue
        params = [] if args in ("", "void") else [parse_param(a, i) for i, a in enumerate(split_args(args))]
        protos.append((name, ret, params))
    return {"handles": handles, "structs": structs, "enums": enums, "defines": defines, "protos": protos}


def split_args(args: str):
    return [a.strip() for a in args.split(",")]


def parse_param(decl: str, index: int):
    """-> (name, c type without the name, array length or None)"""
    array = None
    m = re.search(r"\[(\d*)\]\s*$", decl)
    if m:
        array = m.group(1) or ""
        decl = decl[:m.start()].strip()
    m = re.match(r"^(.*?)(\w+)$", decl)
    ctype, name = m.group(1).strip(), m.group(2)
    if not ctype or name in SCALARS or name.startswith("sgk_") or name == "const":   # no name given
        ctype, name = decl, f"arg{index}"
    return name, ctype, array


def rust_type(ctype: str, array, handles, struct_names) -> str:
    ctype = ctype.strip()
    depth = ctype.count("*")
    # `const T* const*`: constness of each level, outermost pointer last
    parts = [p.strip() for p in ctype.split("*")]
    base_tokens = parts[0].split()
    base_const = "const" in base_tokens
    base = [t for t in base_tokens if t != "const"][0]
    if base in SCALARS:
        rt = SCALARS[base]
    elif base in handles or base in struct_names:
        rt = camel(base)
    else:
        raise ValueError(f"unknown C type {ctype!r}")
    consts = [base_const] + ["const" in p.split() for p in parts[1:]]
    for level in range(depth):
        rt = ("*const " if consts[level] else "*mut ") + rt
    if array is not None:            # a C array parameter is a pointer to its element
        rt = ("*const " if base_const and depth == 0 else "*mut ") + rt if depth == 0 else rt
    return rt


def render(info) -> str:
    handles, structs = info["handles"], info["structs"]
    struct_names = [n for n, _ in structs]
    out = []
    w = out.append
    w("// ffi.rs: the raw binding of libsgk.so (include/sgk.h), generated by rust/gen_ffi.py.")
    w("// Do not edit by hand: change the header and run the generator.")
    w("//")
    w("// Every prototype of the header is declared here, in the header's order. The safe layer")
    w("// of the crate (FullAttentionMetalState, BlockAwarePrefixCache, ...) keeps its signatures")
    w("// and calls these through `check`, which turns a status code into the crate's InferError.")
    w("#![allow(non_camel_case_types, dead_code, clippy::too_many_arguments)]")
    w("")
    w("use crate::error::InferError;")
    w("")
    w("// ---- status codes and constants ----")
    for name, value in info["enums"]:
        w(f"pub const {name}: i32 = {value};")
    for name, value in info["defines"]:
        value = value.strip()
        m = re.match(r"^\((\d+)u\s*<<\s*(\d+)\)$", value)
        if m:
            w(f"pub const {name}: usize = {m.group(1)} << {m.group(2)};")
        else:
            w(f"pub const {name}: usize = {value};")
    w("")
    w("// ---- opaque handles (only ever used behind a pointer) ----")
    for h in handles:
        w("#[repr(C)]")
        w(f"pub struct {camel(h)} {{")
        w("    _private: [u8; 0],")
        w("}")
    w("")
    w("// ---- plain structs passed by pointer ----")
    for name, fields in structs:
        w("#[repr(C)]")
        w("#[derive(Clone, Copy, Debug)]")
        w(f"pub struct {camel(name)} {{")
        for fname, ctype in fields:
            w(f"    pub {fname}: {rust_type(ctype, None, handles, struct_names)},")
        w("}")
    w("")
    w('#[link(name = "sgk")]')
    w('extern "C" {')
    for name, ret, params in info["protos"]:
        args = []
        for pname, ctype, array in params:
            if pname in RUST_KEYWORDS:
                pname += "_"
            args.append(f"{pname}: {rust_type(ctype, array, handles, struct_names)}")
        ret = ret.strip()
        rret = "" if ret == "void" else " -> " + rust_type(ret, None, handles, struct_names)
        w(f"    pub fn {name}({', '.join(args)}){rret};")
    w("}")
    w("")
    w("/// Status of a libsgk call as the crate's error type (src/error.rs:12-75 of the reference).")
    w("pub fn check(rc: i32) -> Result<(), InferError> {")
    w("    if rc == SGK_OK {")
    w("        return Ok(());")
    w("    }")
    w("    // SAFETY: sgk_last_error returns a NUL-terminated thread-local string owned by the library.")
    w("    let msg = unsafe { std::ffi::CStr::from_ptr(sgk_last_error()) }.to_string_lossy().into_owned();")
    w("    Err(match rc {")
    w("        SGK_ERR_DIMENSION => InferError::Dimension(msg),")
    w("        SGK_ERR_CONFIG => InferError::Config(msg),")
    w("        SGK_ERR_MEMORY_GUARD => InferError::MemoryGuard(msg),")
    w("        SGK_ERR_SHAPE => InferError::Shape(msg),")
    w("        // SGK_ERR_BACKEND and SGK_ERR_TIMEOUT: the variant the Metal backend's failures use")
    w("        _ => InferError::Metal(msg),")
    w("    })")
    w("}")
    return "\n".join(out) + "\n"


def main() -> int:
    text = render(parse())
    if "--check" in sys.argv:
        current = open(OUT).read() if os.path.exists(OUT) else ""
        if current != text:
            sys.stderr.write("rust/ffi.rs is out of date: run python rust/gen_ffi.py\n")
            return 1
        return 0
    with open(OUT, "w") as f:
        f.write(text)
    print(f"wrote {OUT}: {text.count('pub fn sgk_')} functions")
    return 0


if __name__ == "__main__":
    sys.exit(main())
