"""`quantize()`: bf16 -> NVFP4 / per-token FP8-E4M3 / per-token INT8 on B200.

Same call signature, output shapes and return tuples as the reference's
python/ac4k_kernel/ops/quant.py:245-294 (shape inference :96-128, :143-171, :187-235).
The global scale that the reference computes with a Triton kernel (:21-59) comes from a
CUDA reduction in the C-ABI library.  One keyword-only extension: `sf_layout="128x4"` makes
the NVFP4 scales come out as [.., ceil(M/128), ceil(K/64), 32, 4, 4] tiles, the layout
tensor memory takes without a shuffle; the default "ac4k" is the reference's layout.
"""
import torch

from .utils import align_up, ceil_div
from .. import _cuda_ops

quantize_nvfp4 = _cuda_ops.quantize_nvfp4
quantize_fp8 = _cuda_ops.quantize_fp8
quantize_int8 = _cuda_ops.quantize_int8

BLOCK_SIZE = 16
PACK_SF = 4
FLOAT4_E2M1_MAX = 6.0
FLOAT8_E4M3_MAX = 448.0


def _global_scale(x: torch.Tensor, max_scale: float) -> torch.Tensor:
    """0-dim fp32 tensor max|x| / max_scale on x's device (quant.py:49-59)."""
    out = torch.empty((), dtype=torch.float32, device=x.device)
    _cuda_ops.global_scale_bf16(out, x if x.is_contiguous() else x.contiguous(), max_scale)
    return out


def _leading(shape, cross_dim, reduce_dim):
    return [shape[i] for i in range(len(shape)) if i != cross_dim and i != reduce_dim]


def _rowwise(input, cross_dim, reduce_dim, max_scale, swizzle, output, sf, out_dtype,
             scale_dtype, default_max, kernel):
    lead = _leading(input.shape, cross_dim, reduce_dim)
    if output is None:
        output = torch.empty(lead + [input.shape[cross_dim], align_up(input.shape[reduce_dim], 16)],
                             dtype=out_dtype, device=input.device)
    if sf is None:
        sf = torch.empty(lead + [align_up(input.shape[cross_dim], 16)], dtype=torch.float32,
                         device=input.device)
    if max_scale is None:
        max_scale = default_max
    max_scale = torch.full([], max_scale, dtype=scale_dtype, device=input.device)
    if swizzle is None:
        kernel(output, sf, input, max_scale, cross_dim, reduce_dim)
    else:
        kernel(output, sf, input, max_scale, cross_dim, reduce_dim, swizzle)
    return output, sf


class Ac4kQuantizeOp(torch.nn.Module):

    def forward(self, input, cross_dim, reduce_dim, max_scale=None, precision="nvfp4",
                swizzle=False, output=None, sf=None, *, sf_layout="ac4k"):
        assert input.ndim >= 2 and input.ndim <= 4, "input tensor must be 2D, 3D or 4D"
        assert precision in ["nvfp4", "fp8e4m3", "int8"]
        if cross_dim < 0:
            cross_dim += input.ndim
        if reduce_dim < 0:
            reduce_dim += input.ndim
        assert cross_dim != reduce_dim, "cross_dim and reduce_dim must be different"

        if precision == "fp8e4m3":
            return _rowwise(input, cross_dim, reduce_dim, max_scale, swizzle, output, sf,
                            torch.float8_e4m3fn, torch.float32, 448, quantize_fp8)
        if precision == "int8":
            return _rowwise(input, cross_dim, reduce_dim, max_scale, None, output, sf,
                            torch.int8, torch.int32, 127, quantize_int8)

        assert sf_layout in ("ac4k", "128x4")
        if max_scale is None:
            max_scale = FLOAT8_E4M3_MAX * FLOAT4_E2M1_MAX
        global_scale = _global_scale(input, float(max_scale))
        lead = _leading(input.shape, cross_dim, reduce_dim)
        m, k = input.shape[cross_dim], input.shape[reduce_dim]
        kp = align_up(k, BLOCK_SIZE * PACK_SF)
        if output is None:
            output = torch.empty(lead + [m, kp // 2], dtype=torch.uint8, device=input.device)
        if sf is None:
            if sf_layout == "ac4k":
                sf_shape = lead + [kp // 64, align_up(m, 16), 4]
            else:
                sf_shape = lead + [ceil_div(m, 128), kp // 64, 32, 4, 4]
            sf = torch.empty(sf_shape, dtype=torch.float8_e4m3fn, device=input.device)
        quantize_nvfp4(output, sf, input, global_scale, cross_dim, reduce_dim, swizzle)
        return output, sf, global_scale


_OP = Ac4kQuantizeOp()


def quantize(input, cross_dim, reduce_dim, max_scale=None, precision="nvfp4", swizzle=False,
             output=None, sf=None, *, sf_layout="ac4k"):
    """Quantize a bf16 tensor to nvfp4, fp8e4m3 or int8.

    Arguments and returns as in the reference (python/ac4k_kernel/ops/quant.py:253-284):
      nvfp4   -> (out u8 [.., M, align_up(K,64)//2], sf e4m3 [.., ceil(K/64), align_up(M,16), 4],
                  global_scale fp32 0-dim)
      fp8e4m3 -> (out e4m3 [.., M, align_up(K,16)], sf fp32 [.., align_up(M,16)])
      int8    -> (out int8 [.., M, align_up(K,16)], sf fp32 [.., align_up(M,16)])
    `max_scale` defaults to 6*448, 448 and 127.  `swizzle` permutes the reduce dim in groups
    of 32 ([4,4,2] -> (1,0,2)) for nvfp4 and of 16 ([2,4,2] -> (1,0,2)) for fp8e4m3.
    """
    return _OP(input, cross_dim, reduce_dim, max_scale=max_scale, precision=precision,
               swizzle=swizzle, output=output, sf=sf, sf_layout=sf_layout)
