"""quantize, linear, attention, rope3d: mirrors python/ac4k_kernel/ops/__init__.py (SparseLinearAttention, a
Triton/PyTorch module on top of `attention`, is not part of this package)."""
from .attention import attention
from .linear import linear, linear_nvfp4, linear_requant
from .rope_3d import rope3d
from .quant import quantize, quantize_nvfp4, quantize_fp8, quantize_int8

__all__ = ["quantize", "linear", "attention", "rope3d", "quantize_nvfp4", "quantize_fp8", "quantize_int8", "linear_nvfp4", "linear_requant"]
