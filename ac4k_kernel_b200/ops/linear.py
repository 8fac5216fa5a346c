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
