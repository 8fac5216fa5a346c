"""`attention()`: softmax(q k^T / sqrt(D)) v with NVFP4, or INT8 (q, k) x FP8 (p, v), operands on B200.

Same signature as the reference's python/ac4k_kernel/ops/attention.py:196-238.  For "nvfp4" the three quantiser
calls are the reference's (attention.py:113-118: q and k along the head dimension, v along the keys with the K
permutation), except that block scales are requested in the tiled layout tensor memory takes.  For "int8+fp8e4m3"
the steps are the reference's as well (attention.py:141-193): the mean over the tokens is taken off k, q and k are
quantised to INT8 in blocks of 64 and 128 tokens (a CUDA kernel here, Triton there), v to FP8 per channel with
max_scale 2.25 and the K permutation.
"""
import math

import torch

from .. import _cuda_ops
from .quant import quantize

mha_nvfp4_fwd = _cuda_ops.mha_nvfp4_fwd
mha_int8_x_fp8_fwd = _cuda_ops.mha_int8_x_fp8_fwd


def _int8_quantize(x, layout, dim, type="token", BLOCK_SIZE=64, HDIM_ALIGN=16, sub=None):
    """(int8 [B, H, N, align_up(D, 16)], fp32 scale [B, H, ceil(N / BLOCK_SIZE)]) as the reference's helper of the
    same name (attention.py:51-99).  `sub` (one token per head, x's layout): x - sub is quantised, bit for bit what
    quantising the bf16 tensor `x - sub` gives."""
    assert HDIM_ALIGN == 16, "HDIM_ALIGN other than 16 is not built"
    assert type == "token", "Only support token quantization yet."
    assert BLOCK_SIZE >= 16 and (BLOCK_SIZE & (BLOCK_SIZE - 1)) == 0
    assert layout in ["BNHD", "BHND"], "Unsupported layout: {}".format(layout)
    if layout == "BNHD":
        B, N, H, D = x.shape
        assert dim in [1, 3]
    else:
        B, H, N, D = x.shape
        assert dim in [2, 3]
    scale = torch.empty([B, H, (x.shape[dim] + BLOCK_SIZE - 1) // BLOCK_SIZE], device=x.device, dtype=torch.float32)
    y = torch.empty([B, H, N, (D + 15) // 16 * 16], device=x.device, dtype=torch.int8)
    _cuda_ops.quantize_int8_block(y, scale, x, layout, BLOCK_SIZE, sub)
    return y, scale


def _int8_x_fp8_attention(q, k, v, layout, Q_QUANTIZE_BLOCK_SIZE=64, K_QUANTIZE_BLOCK_SIZE=128, out=None):
    assert layout in ["BNHD", "BHND"], f"Unsupported layout: {layout}"
    B, Dqk = q.shape[0], q.shape[-1]
    Dv = v.shape[-1]
    if layout == "BNHD":
        Nq, H = q.shape[1], q.shape[2]
    else:
        H, Nq = q.shape[1], q.shape[2]
    n_dim = 1 if layout == "BNHD" else 2
    # k - mean(k): softmax is invariant to it and it shrinks the range INT8 has to cover (attention.py:157); the
    # subtraction happens inside the K quantiser
    k_mean = k.mean(dim=n_dim, keepdim=True)
    q_int8, q_sf = _int8_quantize(q, layout, n_dim, BLOCK_SIZE=Q_QUANTIZE_BLOCK_SIZE)
    k_int8, k_sf = _int8_quantize(k, layout, n_dim, BLOCK_SIZE=K_QUANTIZE_BLOCK_SIZE, sub=k_mean)
    v_fp8, v_sf = quantize(v, 3, n_dim, swizzle=True, max_scale=2.25, precision="fp8e4m3")
    if out is None:
        out_shape = (B, Nq, H, Dv) if layout == "BNHD" else (B, H, Nq, Dv)
        out = torch.empty(out_shape, dtype=torch.bfloat16, device=q.device)
    view = out.permute(0, 2, 1, 3) if layout == "BNHD" else out
    mha_int8_x_fp8_fwd(view, q_int8, q_sf, Q_QUANTIZE_BLOCK_SIZE, k_int8, k_sf, K_QUANTIZE_BLOCK_SIZE, v_fp8, v_sf,
                       1 / math.sqrt(Dqk))
    return out


def _nvfp4_attention(q, k, v, layout, out=None):
    assert layout in ["BNHD", "BHND"], f"Unsupported layout: {layout}"
    B, Dqk = q.shape[0], q.shape[-1]
    Dv = v.shape[-1]
    if layout == "BNHD":
        Nq, H = q.shape[1], q.shape[2]
    else:
        H, Nq = q.shape[1], q.shape[2]
    n_dim = 1 if layout == "BNHD" else 2
    q_fp4, q_sf, q_alpha = quantize(q, n_dim, 3, sf_layout="128x4")
    k_fp4, k_sf, k_alpha = quantize(k, n_dim, 3, sf_layout="128x4")
    v_fp4, v_sf, v_alpha = quantize(v, 3, n_dim, swizzle=True, sf_layout="128x4")
    if out is None:
        out_shape = (B, Nq, H, Dv) if layout == "BNHD" else (B, H, Nq, Dv)
        out = torch.empty(out_shape, dtype=torch.bfloat16, device=q.device)
    view = out.permute(0, 2, 1, 3) if layout == "BNHD" else out      # the kernel addresses [B, H, N, D] by strides
    mha_nvfp4_fwd(view, q_fp4, q_sf, q_alpha, k_fp4, k_sf, k_alpha, v_fp4, v_sf, v_alpha,
                  1 / math.sqrt(Dqk))
    return out


def attention(q, k, v, *, layout="BNHD", precision="int8+fp8e4m3", out=None):
    """q, k: [B, N, H, Dqk] or [B, H, N, Dqk] bf16; v: same with Dv; returns bf16 in q's layout.
    Keyword-only options and defaults of the reference (attention.py:196-204)."""
    assert layout in ["BNHD", "BHND"], f"Unsupported layout: {layout}"
    assert precision in ["nvfp4", "int8+fp8e4m3"], f"Unsupported precision: {precision}"
    assert q.ndim == 4 and k.ndim == 4 and v.ndim == 4
    if precision == "nvfp4":
        return _nvfp4_attention(q, k, v, layout, out=out)
    return _int8_x_fp8_attention(q, k, v, layout, out=out)
