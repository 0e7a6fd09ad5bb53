"""ctypes binding of libqgemm.so (the C-ABI declared in include/qgemm.h).

The reference calls its compiled operators the same way: a ctypes-loaded shared object whose entry
point receives raw device pointers and a stream handle
(tilelang/jit/adapter/cython/cython_wrapper.pyx:143-197, tilelang/jit/adapter/libgen.py:94-104).

There is no fallback: if the library is missing or a call is rejected, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
import threading

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("QGEMM_LIB") or os.path.join(PKG, "libqgemm.so")  # QGEMM_LIB: another build of the library

DT_F16, DT_BF16, DT_I32 = 0, 1, 2
B_KN, B_NK = 0, 1

STATUS_NAMES = {0: "ok", 1: "timeout in TMA producer", 2: "timeout in MMA issuer", 3: "timeout in epilogue",
                4: "timeout in dequant warps", 5: "timeout while draining copies",
                6: "a peer's signal did not arrive"}

# name -> (restype, argtypes); must list every symbol that include/qgemm.h declares.
_c = ctypes
SIGNATURES = {
    "qgemm_version": (_c.c_int, []),
    "qgemm_init": (_c.c_int, []),
    "qgemm_last_error": (_c.c_char_p, []),
    "qgemm_set_wait_limit_ms": (None, [_c.c_uint32]),
    "qgemm_debug_withhold_commit": (None, [_c.c_int]),
    "qgemm_w8a8": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                              _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64,
                              _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "qgemm_w8a8_grouped": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                      _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64,
                                      _c.c_int64, _c.c_int64, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "qgemm_w4a16_workspace_bytes": (_c.c_int64, [_c.c_int64, _c.c_int64, _c.c_int64]),
    "qgemm_w4a16_counter_bytes": (_c.c_int64, []),
    "qgemm_w4a16": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p,
                               _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
                               _c.c_void_p, _c.c_void_p]),
    "qgemm_w4a16_batched_workspace_bytes": (_c.c_int64, [_c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64]),
    "qgemm_w4a16_batched": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p,
                                       _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64,
                                       _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "qgemm_w4a16_ex_workspace_bytes": (_c.c_int64, [_c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int]),
    "qgemm_w4a16_ex": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int,
                                  _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64,
                                  _c.c_int64, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "qgemm_w4a16_gather": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_int,
                                      _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64,
                                      _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "qgemm_ipc_export": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p]),
    "qgemm_ipc_open": (_c.c_int, [_c.c_void_p, _c.c_void_p]),
    "qgemm_ipc_close": (_c.c_int, [_c.c_void_p]),
    "qgemm_peer_signal_wait": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p, _c.c_uint32, _c.c_void_p, _c.c_void_p,
                                          _c.c_void_p]),
    "qgemm_w4a16_noalloc": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p,
                                       _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int, _c.c_void_p,
                                       _c.c_void_p]),
    "qgemm_unpack_int4": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int, _c.c_void_p]),
    "qgemm_w4a8": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64,
                              _c.c_int64, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "qgemm_w4a8_act_quant": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int,
                                        _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "qgemm_act_quant": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
                                   _c.c_void_p]),
}

_lock = threading.Lock()
_lib = None


class QGemmError(RuntimeError):
    """A call into libqgemm.so was rejected, or a kernel reported an expired wait."""


def load() -> ctypes.CDLL:
    """Load libqgemm.so (building it first when a compiler is present and it is stale or missing)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if os.environ.get("QGEMM_NO_BUILD") != "1" and not os.environ.get("QGEMM_LIB"):
            try:
                from . import build as _build
                if _build.needs_build():
                    _build.build()
            except Exception:
                if not os.path.isfile(LIB_PATH):
                    raise
        if not os.path.isfile(LIB_PATH):
            raise QGemmError(f"{LIB_PATH} not found: build it with `python -m tilelang_ascend_b200.build`")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


def last_error() -> str:
    msg = load().qgemm_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, what: str):
    if rc != 0:
        raise QGemmError(f"{what}: {last_error()}")
