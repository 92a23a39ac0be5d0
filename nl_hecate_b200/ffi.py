"""ctypes loader for libnlh_b200.so.

Prototypes are derived from ``include/nlh_ffi.h`` so that the header is the
single source of truth for the C ABI. Loading fails loudly when the library is
missing: there is no CPU fallback in this package.
"""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnlh_b200.so")
HEADER = os.path.join(os.path.dirname(HERE), "include", "nlh_ffi.h")

NLH_OK = 0

_SCALARS = {
    "int32_t": C.c_int32, "int64_t": C.c_int64, "uint32_t": C.c_uint32, "uint64_t": C.c_uint64,
    "float": C.c_float,
    "int": C.c_int,
}


class AdamWTensorDesc(C.Structure):
    """Mirror of ``nlh_adamw_tensor_desc`` (include/nlh_ffi.h)."""
    _fields_ = [("bc1_inv", C.c_float), ("bc2_inv", C.c_float), ("weight_decay", C.c_float),
                ("lr_scale", C.c_float), ("clamp_lo", C.c_float), ("clamp_hi", C.c_float),
                ("has_clamp", C.c_int32), ("active", C.c_int32)]


def _ctype(decl: str):
    decl = decl.strip()
    if decl == "void":
        return None
    if "*" in decl:
        return C.c_char_p if decl.replace(" ", "") == "constchar*" else C.c_void_p
    base = decl.replace("const", "").split()[0]
    return _SCALARS[base]


def parse_header(path: str = HEADER):
    """Returns {name: (restype, [argtypes], [argnames])} for every prototype in the header."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    text = re.sub(r"typedef struct.*?\}\s*\w+\s*;", "", text, flags=re.S)
    text = re.sub(r"^\s*#[^\n]*", "", text, flags=re.M)
    text = text.replace('extern "C" {', "")
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(\w+)\s*\(([^()]*)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if name in ("defined",) or ret.startswith("#"):
            continue
        argtypes, argnames = [], []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                mm = re.match(r"(.*?)(\w+)$", a)
                argtypes.append(_ctype(mm.group(1)))
                argnames.append(mm.group(2))
        protos[name] = (_ctype(ret), argtypes, argnames)
    return protos


_lib = None


def lib() -> C.CDLL:
    """The loaded library with argtypes/restypes set. Raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m nl_hecate_b200.build` "
                "(there is no CPU fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (ret, argtypes, _) in parse_header().items():
            fn = getattr(handle, name)   # AttributeError if the header and library disagree
            fn.restype = ret
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, where: str) -> None:
    if status != NLH_OK:
        err = lib().nlh_last_error()
        lib().nlh_clear_status()   # the recorded status is sticky: do not leak it into later calls
        raise RuntimeError(f"{where} failed with status {status}: {err.decode() if err else ''}")


def check_void(where: str) -> None:
    """After a void drop-in entry: raise if it recorded an error."""
    st = lib().nlh_last_status()
    if st != NLH_OK:
        err = lib().nlh_last_error()
        lib().nlh_clear_status()
        raise RuntimeError(f"{where} failed with status {st}: {err.decode() if err else ''}")
