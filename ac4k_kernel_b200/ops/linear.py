"""`linear()`: y = x @ weight.T + bias with NVFP4 operands on B200.

Same signature as the reference's python/ac4k_kernel/ops/linear.py:41-75.  Scale tensors
may be in either NVFP4 scale layout (rank 3 = the reference's, rank 5 = 128x4 tiles), as
long as both operands use the same one.
"""
import torch

from .. import _cuda_ops

linear_nvfp4 = _cuda_ops.linear_nvfp4


class Ac4kLinearOp(torch.nn.Module):

    def forward(self, x, x_scale, x_global_scale, weight, weight_scale, weight_global_scale,
                bias, out=None):
        if (bias is not None) and (bias.ndim == 1):
            bias = bias.reshape(1, -1)
        if out is None:
            m, n = x.shape[0], weight.shape[0]
            out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        linear_nvfp4(out, x, x_scale, x_global_scale, weight, weight_scale,
                     weight_global_scale, bias)
        return out


_OP = Ac4kLinearOp()


def linear(x, x_scale, x_global_scale, weight, weight_scale, weight_global_scale, bias=None,
           out=None):
    """x: packed nvfp4 [M, K/2] u8; weight: packed nvfp4 [N, K/2] u8; *_scale: e4m3 block
    scales; *_global_scale: fp32 0-dim; bias: [N] or [1, N] bf16/fp16/fp32; out: optional
    [M, N] bf16/fp16/fp32 (bf16 when allocated here).  Returns out."""
    return _OP(x, x_scale, x_global_scale, weight, weight_scale, weight_global_scale, bias,
               out=out)


def linear_requant(x, x_scale, x_global_scale, weight, weight_scale, weight_global_scale,
                   out_global_scale, bias=None, sf_layout="128x4"):
    """`linear()` followed by `quantize(..., global_scale=out_global_scale)` in one kernel: the GEMM's
    epilogue rounds the result to bf16 and quantises it to NVFP4 (blocks of 16 along N), so the output
    can feed the next `linear()` directly.  Bit-identical to the two-call sequence; the reference has
    no counterpart.  Returns (packed [M, N/2] u8, block scales in `sf_layout`, out_global_scale)."""
    from .utils import align_up, ceil_div
    if (bias is not None) and (bias.ndim == 1):
        bias = bias.reshape(1, -1)
    m, n = x.shape[0], weight.shape[0]
    out = torch.empty((m, n // 2), dtype=torch.uint8, device=x.device)
    if sf_layout == "ac4k":
        sf_shape = (n // 64, align_up(m, 16), 4)
    elif sf_layout == "128x4":
        sf_shape = (ceil_div(m, 128), n // 64, 32, 4, 4)
    else:
        raise ValueError(f"unknown sf_layout {sf_layout!r}")
    out_sf = torch.empty(sf_shape, dtype=torch.float8_e4m3fn, device=x.device)
    _cuda_ops.linear_nvfp4_requant(out, out_sf, out_global_scale, x, x_scale, x_global_scale, weight,
                                   weight_scale, weight_global_scale, bias)
    return out, out_sf, out_global_scale
