"""`attention()`: softmax(q k^T / sqrt(D)) v with NVFP4 operands on B200.

Same signature as the reference's python/ac4k_kernel/ops/attention.py:196-238 for
`precision="nvfp4"` (the int8+fp8e4m3 precision is a different kernel family and raises
NotImplementedError here).  The three quantiser calls are the reference's
(attention.py:113-118: q and k along the head dimension, v along the keys with the K
permutation), except that block scales are requested in the tiled layout tensor memory takes.
"""
import math

import torch

from .. import _cuda_ops
from .quant import quantize

mha_nvfp4_fwd = _cuda_ops.mha_nvfp4_fwd


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
    Keyword-only options and defaults of the reference (attention.py:196-204); only precision="nvfp4" is built."""
    assert layout in ["BNHD", "BHND"], f"Unsupported layout: {layout}"
    assert precision in ["nvfp4", "int8+fp8e4m3"], f"Unsupported precision: {precision}"
    assert q.ndim == 4 and k.ndim == 4 and v.ndim == 4
    if precision != "nvfp4":
        raise NotImplementedError("attention(precision='int8+fp8e4m3') is outside what this sm100 build covers; "
                                  "pass precision='nvfp4'")
    return _nvfp4_attention(q, k, v, layout, out=out)
