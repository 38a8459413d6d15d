"""The Rust binding a maintainer drops into the reference crate (rust/ffi.rs) declares every
prototype of include/sgk.h with the same arity and the same integer / float widths. No Rust
toolchain exists here, so the file is checked against the header instead of being compiled."""
import ctypes as C
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from saragossa_b200 import _ffi  # noqa: E402

FFI_RS = os.path.join(ROOT, "rust", "ffi.rs")

_RUST_SCALARS = {
    "i32": C.c_int32, "i64": C.c_int64, "u64": C.c_uint64, "u32": C.c_uint32, "usize": C.c_size_t,
    "f32": C.c_float, "f64": C.c_double, "std::os::raw::c_int": C.c_int,
}


def _rust_protos():
    text = open(FFI_RS).read()
    block = text[text.index('extern "C" {'):]
    block = block[:block.index("\n}\n")]
    protos = {}
    for m in re.finditer(r"pub fn (sgk_\w+)\((.*?)\)( -> (.*?))?;", block):
        name, args, ret = m.group(1), m.group(2).strip(), m.group(4)
        params = []
        if args:
            for a in args.split(", "):
                pname, ptype = a.split(": ", 1)
                params.append(ptype)
        protos[name] = (ret, params)
    return protos


def _as_ctype(rust: str, is_ret: bool):
    if rust is None:
        return None
    if rust.startswith("*"):
        return C.c_char_p if is_ret and rust.endswith("c_char") else C.c_void_p
    return _RUST_SCALARS[rust]


def test_ffi_rs_declares_every_prototype_with_matching_widths():
    header = _ffi.parse_header()
    rust = _rust_protos()
    assert sorted(rust) == sorted(header)
    for name, (res, args) in header.items():
        r_ret, r_args = rust[name]
        assert _as_ctype(r_ret, True) == res, name
        assert len(r_args) == len(args), name
        for i, (ra, ha) in enumerate(zip(r_args, args)):
            assert _as_ctype(ra, False) == ha, (name, i, ra)


def test_ffi_rs_is_what_the_generator_gives():
    done = subprocess.run([sys.executable, os.path.join(ROOT, "rust", "gen_ffi.py"), "--check"],
                          capture_output=True, text=True)
    assert done.returncode == 0, done.stderr


def test_ffi_rs_maps_every_status_code():
    text = open(FFI_RS).read()
    header = open(os.path.join(ROOT, "include", "sgk.h")).read()
    for code in re.findall(r"\b(SGK_ERR_\w+)\s*=", header):
        assert f"pub const {code}: i32" in text, code
    for variant in ("Dimension", "Config", "MemoryGuard", "Shape", "Metal"):
        assert f"InferError::{variant}" in text


def test_build_rs_compiles_for_sm_100a_and_links_the_library():
    text = open(os.path.join(ROOT, "rust", "build.rs")).read()
    assert "arch=compute_100a,code=sm_100a" in text
    assert "cargo:rustc-link-lib=dylib=sgk" in text
