"""ctypes binding of libsgk.so, generated from include/sgk.h.

The header is the single source of truth: every `sgk_*` prototype in it is
parsed into a ctypes signature (pointers become void*, so numpy arrays and
device addresses are passed as integers). Loading fails loudly when the library
is missing or lacks a declared symbol; there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(os.path.dirname(HERE), "include", "sgk.h")
LIB_PATH = os.environ.get("SGK_LIB") or os.path.join(HERE, "_lib", "libsgk.so")

_SCALARS = {
    "int32_t": C.c_int32, "int64_t": C.c_int64, "uint64_t": C.c_uint64, "uint32_t": C.c_uint32,
    "size_t": C.c_size_t, "float": C.c_float, "int": C.c_int, "double": C.c_double,
}


def parse_header(path: str = HEADER):
    """Returns {name: (restype, [argtypes])} for every sgk_* prototype."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"#[^\n]*", " ", text)
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(sgk_\w+)\s*\(([^;{}]*?)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if ret.startswith("typedef") or "struct" in ret:
            continue
        protos[name] = (_ctype(ret, True), [] if args in ("", "void") else [_ctype(a, False) for a in args.split(",")])
    return protos


def _ctype(decl: str, is_ret: bool):
    decl = decl.strip()
    if "*" in decl or "[" in decl:
        if is_ret and "char" in decl:
            return C.c_char_p
        return C.c_void_p
    base = [t for t in decl.replace("const", " ").split() if t]
    # drop the parameter name when present
    for tok in base:
        if tok in _SCALARS:
            return _SCALARS[tok]
    if base and base[0] == "void":
        return None
    raise ValueError(f"cannot map C declaration {decl!r}")


_lib = None


def lib() -> C.CDLL:
    """Loads libsgk.so (building it first if the sources are newer)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from . import build as _build
        _build.build()
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: run `python -m saragossa_b200.build` (there is no fallback path)")
    handle = C.CDLL(LIB_PATH)
    missing = []
    for name, (res, args) in parse_header().items():
        try:
            fn = getattr(handle, name)
        except AttributeError:
            missing.append(name)
            continue
        fn.restype = res
        fn.argtypes = args
    if missing:
        raise RuntimeError(f"libsgk.so lacks symbols declared in sgk.h: {missing}")
    _lib = handle
    return _lib


def last_error() -> str:
    msg = lib().sgk_last_error()
    return msg.decode() if msg else ""
