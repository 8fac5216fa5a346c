"""ctypes loader for the C-ABI library `libac4k_b200.so` (declared in include/ac4k_b200.h).

There is no CPU fallback: if the library is missing or fails to load, importing the
package raises.  Build it with `python ac4k_kernel_b200/build.py`.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libac4k_b200.so")

_c_i64p = ctypes.POINTER(ctypes.c_int64)
_vp = ctypes.c_void_p

# name -> (restype, argtypes); must list every symbol of include/ac4k_b200.h
SIGNATURES = {
    "ac4k_arch": (ctypes.c_char_p, []),
    "ac4k_arch_description": (ctypes.c_char_p, []),
    "ac4k_backend": (ctypes.c_char_p, []),
    "ac4k_version": (ctypes.c_char_p, []),
    "ac4k_last_error": (ctypes.c_char_p, []),
    "ac4k_device_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint32), ctypes.c_int]),
    "ac4k_global_scale_bf16": (ctypes.c_int, [_vp, ctypes.c_int64, ctypes.c_float, _vp, _vp]),
    "ac4k_quantize_nvfp4": (ctypes.c_int, [_vp, _vp, _vp, _vp, _c_i64p, _c_i64p, ctypes.c_int,
                                           ctypes.c_int, _vp]),
    "ac4k_quantize_fp8": (ctypes.c_int, [_vp, _vp, _vp, _vp, _c_i64p, _c_i64p, ctypes.c_int, _vp]),
    "ac4k_quantize_int8": (ctypes.c_int, [_vp, _vp, _vp, _vp, _c_i64p, _c_i64p, _vp]),
    "ac4k_linear_nvfp4": (ctypes.c_int, [_vp, ctypes.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                         ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_int64, ctypes.c_int, _vp]),
    "ac4k_linear_nvfp4_noalloc": (ctypes.c_int, [_vp, ctypes.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                                 ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                                 ctypes.c_int64, ctypes.c_int, _vp]),
    "ac4k_linear_nvfp4_gather": (ctypes.c_int, [ctypes.POINTER(_vp), ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_int,
                                                ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, _vp]),
    "ac4k_linear_nvfp4_requant": (ctypes.c_int, [_vp, _vp, _vp, ctypes.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                                 ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                                 ctypes.c_int, _vp]),
    "ac4k_mha_nvfp4_fwd": (ctypes.c_int, [_vp, _c_i64p, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                          ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                          ctypes.c_int64, ctypes.c_int64, ctypes.c_float, ctypes.c_int, _vp]),
    "ac4k_quantize_int8_block": (ctypes.c_int, [_vp, _vp, _vp, _c_i64p, _c_i64p, ctypes.c_int64, _vp, _c_i64p, _vp]),
    "ac4k_mha_int8_x_fp8_fwd": (ctypes.c_int, [_vp, _c_i64p, _vp, _vp, ctypes.c_int64, _vp, _vp, ctypes.c_int64, _vp, _vp,
                                               ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                               ctypes.c_int64, ctypes.c_int64, ctypes.c_float, _vp]),
    "ac4k_rope3d": (ctypes.c_int, [_vp, _vp, _vp, _vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                   ctypes.c_int64, _vp]),
    "ac4k_peer_alloc": (ctypes.c_int, [ctypes.c_int64, ctypes.POINTER(_vp), ctypes.c_char_p]),
    "ac4k_peer_open": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "ac4k_peer_close": (ctypes.c_int, [_vp]),
    "ac4k_peer_free": (ctypes.c_int, [_vp]),
}


def load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: the sm_100a extension is not built and this package has "
            "no other backend.  Run `python ac4k_kernel_b200/build.py`.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library is stale
        fn.restype = res
        fn.argtypes = args
    return lib


LIB = load()


def last_error() -> str:
    return LIB.ac4k_last_error().decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (code {rc}): {last_error()}")


def device_status(clear: bool = True) -> int:
    """The device status word (0, or the code of an expired device-side wait); synchronises the device."""
    v = ctypes.c_uint32(0)
    rc = LIB.ac4k_device_status(ctypes.byref(v), int(clear))
    if rc != 0 and rc != -7:            # -7 (AC4K_ERR_TIMEOUT) comes with the code in v
        check(rc, "ac4k_device_status")
    return v.value
