"""ctypes binding of libruda_b200.so — the Python stand-in for the Rust FFI crate.

The library is loaded from this package directory.  If it is missing, loading fails loudly: there is
no CPU fallback (rust-ascend src/backend.rs:43-45 makes the same promise).
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libruda_b200.so")


class rb_options(C.Structure):
    _fields_ = [("device", C.c_int32), ("synchronous", C.c_int32), ("reserved", C.c_uint64 * 4)]


class rb_tensor(C.Structure):
    _fields_ = [("handle", C.c_uint64), ("offset", C.c_uint64), ("dtype", C.c_uint32), ("rank", C.c_uint32),
                ("shape", C.c_uint64 * 8), ("strides", C.c_uint64 * 8)]


class rb_stats(C.Structure):
    _fields_ = [("launches", C.c_uint64), ("synchronizations", C.c_uint64), ("empty_calls", C.c_uint64),
                ("bytes_in_use", C.c_uint64), ("allocations", C.c_uint64)]


_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} is missing: build it with `python -m rust_ascend_b200.build` "
                          "(the B200 backend has no CPU fallback)")
        _lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        _lib.rb_last_error.restype = C.c_char_p
    return _lib


def declared_symbols(header_path: str) -> list[str]:
    """Names of every RB_API function the public header declares."""
    import re
    text = open(header_path).read()
    return re.findall(r"RB_API\s+[A-Za-z_0-9\* ]+?\s+\**(rb_[a-z0-9_]+)\s*\(", text)
