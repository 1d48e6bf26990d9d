"""ctypes binding of the C-ABI library ``libspeed3r_b200.so`` (declared in include/speed3r_b200.h).

There is no fallback: if the library is missing and cannot be built, or a call returns an error,
a ``RuntimeError`` is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libspeed3r_b200.so")

_i, _i64, _f, _p, _sz = C.c_int, C.c_int64, C.c_float, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); must list every function the header declares
SIGNATURES = {
    "s3r_version": (_i, []),
    "s3r_last_error": (_i, [C.c_char_p, _i]),
    "s3r_device_status": (_i, [C.POINTER(C.c_uint32), _i]),
    "s3r_pool_fwd": (_i, [_p, _i64, _i64, _i64, _p, _i, _i, _i, _i, _i, _i, _p]),
    "s3r_pool_bwd": (_i, [_p, _p, _i64, _i64, _i64, _i, _i, _i, _i, _i, _i, _i, _p]),
    "s3r_qkv_prologue_fwd": (_i, [_p, _p, _p, _p, _i, _p, _p, _p, _p, _f, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "s3r_cmp_attn_topk_fwd": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _p]),
    "s3r_cmp_attn_blocktopk_fwd": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _i, _p]),
    "s3r_cmp_attn_bwd": (_i, [_p] * 10 + [_i, _i, _i, _i, _i, _f, _p]),
    "s3r_sel_attn_fwd": (_i, [_p, _p, _p, _i, _i64, _p, _p, _p, _p, _i64, _i64, _i64, _p, _p,
                              _i, _i, _i, _i, _i, _i, _i, _f, _p]),
    "s3r_csr_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "s3r_build_key_csr": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _p, _sz, _p]),
    "s3r_build_key_csr_static": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "s3r_merge_bwd": (_i, [_p, _p, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "s3r_delta": (_i, [_p, _p, _p, _i64, _i, _p]),
    "s3r_sel_attn_bwd": (_i, [_p] * 12 + [_i, _i, _i, _i, _i, _i, _i, _f, _p]),
    "s3r_copy2d_async": (_i, [_p, _sz, _p, _sz, _sz, _sz, _p]),
    "s3r_peer_pull": (_i, [_p, _p, _p, _i, _i, _p]),
    "s3r_ipc_export": (_i, [_p, _p, C.POINTER(C.c_int64)]),
    "s3r_ipc_import": (_i, [_p, _i64, C.POINTER(_p)]),
}

# the tests-only companion library (include/speed3r_b200_check.h); nothing in the package calls it
CHECK_LIB_PATH = os.path.join(_PKG, "libspeed3r_b200_check.so")
CHECK_SIGNATURES = {
    "s3r_check_cmp_attn_topk_fwd": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _p]),
    "s3r_check_sel_attn_fwd": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _p]),
    "s3r_check_wait_gives_up": (_i, [C.c_uint64, _p, _p]),
    "s3r_last_error": (_i, [C.c_char_p, _i]),
    "s3r_device_status": (_i, [C.POINTER(C.c_uint32), _i]),
}

_lock = threading.Lock()
_lib = None
_check_lib = None


def load() -> C.CDLL:
    """Load (building first if the shared object is absent and nvcc is present)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            from . import build as _build
            _build.build()
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


def load_check() -> C.CDLL:
    """The tests-only companion library (device-side cross-checks, the bounded-wait probe)."""
    global _check_lib
    with _lock:
        if _check_lib is None:
            if not os.path.exists(CHECK_LIB_PATH):
                from . import build as _build
                _build.build()
            lib = C.CDLL(CHECK_LIB_PATH)
            for name, (res, args) in CHECK_SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _check_lib = lib
        return _check_lib


def last_error() -> str:
    buf = C.create_string_buffer(512)
    load().s3r_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}: {last_error()}")


def device_status(clear: bool = True) -> int:
    v = C.c_uint32(0)
    check(load().s3r_device_status(C.byref(v), 1 if clear else 0), "s3r_device_status")
    return int(v.value)
