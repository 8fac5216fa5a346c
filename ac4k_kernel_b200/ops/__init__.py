"""quantize, linear, attention, rope3d and the direct kernel entry points: mirrors python/ac4k_kernel/ops/__init__.py:5-27
(SparseLinearAttention, a Triton/PyTorch training module on top of attention, is not part of this package)."""
from .attention import attention, mha_nvfp4_fwd, mha_int8_x_fp8_fwd
from .linear import linear, linear_nvfp4, linear_requant
from .rope_3d import rope3d, rope3d_kernel
from .quant import quantize, quantize_nvfp4, quantize_fp8, quantize_int8

__all__ = [
    # high-level APIs
    "attention", "quantize", "linear", "rope3d",
    # direct kernel access
    "mha_nvfp4_fwd", "mha_int8_x_fp8_fwd", "quantize_nvfp4", "quantize_fp8", "quantize_int8", "linear_nvfp4", "rope3d_kernel",
    # not in the reference: GEMM whose epilogue re-quantises its output to NVFP4
    "linear_requant",
]
