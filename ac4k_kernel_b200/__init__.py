"""ac4k_kernel_b200: the operators of ac4k_kernel written for B200 (sm_100a): the NVFP4 linear path
(quantize -> block-scaled GEMM), NVFP4 and INT8 x FP8 attention, 3-D RoPE.  Layout of this module mirrors
python/ac4k_kernel/__init__.py.

The compiled backend is the C-ABI library `libac4k_b200.so`; importing this package fails
if it is not built (there is no other backend and no CPU fallback).
"""
__version__ = "0.1.0"

from ._cuda_ops import (  # noqa: F401
    __arch__,
    __backend__,
    mha_nvfp4_fwd,
    mha_int8_x_fp8_fwd,
    quantize_nvfp4,
    quantize_fp8,
    quantize_int8,
    linear_nvfp4,
    rope3d,
)

_backend = __backend__
_arch = __arch__


def get_backend():
    """Return the compiled backend ('cuda')."""
    return _backend


def get_arch():
    """Return the compiled architecture ('sm100')."""
    return _arch


def get_info():
    return {"version": __version__, "backend": _backend, "arch": _arch}


__all__ = ["__version__", "get_backend", "get_arch", "get_info", "mha_nvfp4_fwd",
           "mha_int8_x_fp8_fwd", "quantize_nvfp4", "quantize_fp8", "quantize_int8",
           "linear_nvfp4", "rope3d"]
