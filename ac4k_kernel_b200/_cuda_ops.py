"""Drop-in for ac4k_kernel's compiled module `ac4k_kernel._cuda_ops` on B200 (sm_100a).

Same names, argument order and argument checks as the pybind module defined in the
reference's lib/cuda_bindings.cc:37-97 (C++ prototypes in include/ac4k_kernel/ops.h:27-48).
Each function validates its tensors the way the reference's host launcher does, then hands
raw device pointers and the current CUDA stream to the C-ABI library; outputs are
pre-allocated by the caller and written in place.  A failed check raises RuntimeError, as
the reference's TORCH_CHECKs do.

Scale-factor layout is inferred from the rank of `sf`: `in.dim() + 1` is the reference's
[.., K/64, align16(M), 4] layout, `in.dim() + 3` the tensor-memory-ready
[.., ceil(M/128), K/64, 32, 4, 4] tiles.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import LIB, check

__arch__ = LIB.ac4k_arch().decode()
__arch_description__ = LIB.ac4k_arch_description().decode()
__backend__ = LIB.ac4k_backend().decode()
__version__ = LIB.ac4k_version().decode()

SF_AC4K, SF_TILE128X4 = 0, 1
_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_I64x4 = ctypes.c_int64 * 4


def _align_up(a, b):
    return (a + b - 1) // b * b


def _ceil_div(a, b):
    return (a + b - 1) // b


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _check_tensor(x, dtype, name):
    _require(isinstance(x, torch.Tensor), f"{name} must be a tensor")
    _require(x.is_cuda, f"{name} must be a CUDA tensor")
    _require(x.is_contiguous(), f"{name} must be contiguous")
    _require(x.dtype == dtype, f"Inconsistency of Tensor type: {name} must be {dtype}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _view4(inp: torch.Tensor, cross_dim: int, reduce_dim: int):
    """Sizes and element strides ordered [outer0, outer1, cross, reduce], rank padded to 4
    with leading 1s (quantize_nvfp4.cu:226-241)."""
    nd = inp.dim()
    others = [i for i in range(nd) if i not in (cross_dim, reduce_dim)]
    shape = [1] * (2 - len(others)) + [inp.size(i) for i in others]
    stride = [0] * (2 - len(others)) + [inp.stride(i) for i in others]
    shape += [inp.size(cross_dim), inp.size(reduce_dim)]
    stride += [inp.stride(cross_dim), inp.stride(reduce_dim)]
    return shape, stride, others


def _check_quant_common(out, inp, cross_dim, reduce_dim, reduce_align, reduce_div):
    _require(2 <= inp.dim() <= 4, "in must be 2-4D")
    _require(0 <= cross_dim < inp.dim(), "cross_dim must be less than in.dim()")
    _require(0 <= reduce_dim < inp.dim(), "reduce_dim must be less than in.dim()")
    _require(cross_dim != reduce_dim, "cross_dim and reduce_dim must be different")
    _require(out.dim() == inp.dim(), "out must be the same dim as in")
    shape, stride, others = _view4(inp, cross_dim, reduce_dim)
    for c, i in enumerate(others):
        _require(out.size(c) == inp.size(i), "out must be the same shape as in")
    _require(out.size(-2) == shape[2], "meet invalid cross dim size")
    _require(out.size(-1) == _align_up(shape[3], reduce_align) // reduce_div,
             "meet invalid reduce dim size")
    return shape, stride, others


def quantize_nvfp4(out, sf, input, global_scale, cross_dim, reduce_dim, swizzle):
    """bf16 -> NVFP4 (ops.h:27-29; checks of quantize_nvfp4.cu:171-224)."""
    _check_tensor(input, torch.bfloat16, "in")
    _check_tensor(global_scale, torch.float32, "global_scale")
    _require(global_scale.dim() == 0, "global_scale must be a scalar")
    _check_tensor(out, torch.uint8, "out")
    _check_tensor(sf, torch.float8_e4m3fn, "sf")
    shape, stride, others = _check_quant_common(out, input, int(cross_dim), int(reduce_dim), 64, 2)
    nd = input.dim()
    kt = _ceil_div(shape[3], 64)
    if sf.dim() == nd + 1:
        layout = SF_AC4K
        want = [input.size(i) for i in others] + [kt, _align_up(shape[2], 16), 4]
    elif sf.dim() == nd + 3:
        layout = SF_TILE128X4
        want = [input.size(i) for i in others] + [_ceil_div(shape[2], 128), kt, 32, 4, 4]
    else:
        raise RuntimeError("meet invalid sf rank")
    _require(list(sf.shape) == want, "meet invalid sf shape")
    with torch.cuda.device(input.device):
        check(LIB.ac4k_quantize_nvfp4(out.data_ptr(), sf.data_ptr(), input.data_ptr(),
                                      global_scale.data_ptr(), _I64x4(*shape), _I64x4(*stride),
                                      int(bool(swizzle)), layout, _stream(input)),
              "quantize_nvfp4")


def _quantize_rowwise(fn, name, out, sf, input, scale_max, scale_dtype, out_dtype, cross_dim,
                      reduce_dim, swizzle):
    _check_tensor(input, torch.bfloat16, "in")
    _check_tensor(scale_max, scale_dtype, "scale_max")
    _require(scale_max.dim() == 0, "scale_max must be a scalar")
    _check_tensor(out, out_dtype, "out")
    _check_tensor(sf, torch.float32, "sf")
    shape, stride, others = _check_quant_common(out, input, int(cross_dim), int(reduce_dim), 16, 1)
    _require(sf.dim() == input.dim() - 1, "meet invalid sf rank")
    want = [input.size(i) for i in others] + [_align_up(shape[2], 16)]
    _require(list(sf.shape) == want, "meet invalid sf shape")
    args = [out.data_ptr(), sf.data_ptr(), input.data_ptr(), scale_max.data_ptr(),
            _I64x4(*shape), _I64x4(*stride)]
    if swizzle is not None:
        args.append(int(bool(swizzle)))
    with torch.cuda.device(input.device):
        check(fn(*args, _stream(input)), name)


def quantize_fp8(out, sf, input, scale_max, cross_dim, reduce_dim, swizzle):
    """bf16 -> per-row e4m3 (ops.h:31-33; checks of quantize_fp8.cu:196-247)."""
    _quantize_rowwise(LIB.ac4k_quantize_fp8, "quantize_fp8", out, sf, input, scale_max,
                      torch.float32, torch.float8_e4m3fn, cross_dim, reduce_dim, swizzle)


def quantize_int8(out, sf, input, scale_max, cross_dim, reduce_dim):
    """bf16 -> per-row int8, int32 scale_max (ops.h:35-37; quantize_int8.cu:179-230)."""
    _quantize_rowwise(LIB.ac4k_quantize_int8, "quantize_int8", out, sf, input, scale_max,
                      torch.int32, torch.int8, cross_dim, reduce_dim, None)


def linear_nvfp4(D, A, A_sf, A_global_scale, B, B_sf, B_global_scale, bias):
    """D = (A_gs*B_gs) * A @ B^T + bias (ops.h:43-48; checks of linear_nvfp4.cu:759-805)."""
    _require(D.dim() == 2, "d must be a 2d matrix")
    M, N = D.shape
    _require(D.dtype in _DT, "d must be bfloat16, half or float")
    _require(D.is_cuda and D.is_contiguous(), "d must be contiguous")
    _require(A.dim() == 2, "a must be a 2d matrix")
    _check_tensor(A, torch.uint8, "a")
    _require(A.size(0) == M, f"A size(0) must be {M} but see {A.size(0)}")
    K = A.size(1) * 2
    _require(K % 16 == 0, f"A size(1)*2 must be multiple of 16 but see {K}")
    _require(B.dim() == 2, "b must be a 2d matrix")
    _check_tensor(B, torch.uint8, "b")
    _require(B.size(0) == N, f"B size(0) must be {N} but see {B.size(0)}")
    _require(B.size(1) == A.size(1), "B size(1) must equal A size(1)")
    kt = _ceil_div(K, 64)
    _check_tensor(A_sf, torch.float8_e4m3fn, "scale_a")
    _check_tensor(B_sf, torch.float8_e4m3fn, "scale_b")
    if A_sf.dim() == 3:
        layout = SF_AC4K
        _require(list(A_sf.shape) == [kt, _align_up(M, 16), 4], "scale_a has an invalid shape")
        _require(B_sf.dim() == 3, "scale_b must be a 3d matrix")
        _require(list(B_sf.shape) == [kt, _align_up(N, 16), 4], "scale_b has an invalid shape")
    elif A_sf.dim() == 5:
        layout = SF_TILE128X4
        _require(list(A_sf.shape) == [_ceil_div(M, 128), kt, 32, 4, 4], "scale_a has an invalid shape")
        _require(list(B_sf.shape) == [_ceil_div(N, 128), kt, 32, 4, 4], "scale_b has an invalid shape")
    else:
        raise RuntimeError("scale_a must be a 3d matrix")
    _check_tensor(A_global_scale, torch.float32, "global_scale_a")
    _require(A_global_scale.dim() == 0, "A_global_scale must be a scalar")
    _check_tensor(B_global_scale, torch.float32, "global_scale_b")
    _require(B_global_scale.dim() == 0, "B_global_scale must be a scalar")
    bias_ptr, bias_dt = None, 0
    if bias is not None:
        _require(bias.dtype in _DT, "bias must be bfloat16, half or float")
        _require(bias.is_cuda and bias.is_contiguous(), "bias must be contiguous")
        _require(bias.dim() == 2, "bias must be a 2d matrix")
        _require(bias.size(0) == 1, "bias shape[0] must be 1")
        _require(bias.size(1) == N, f"bias shape[1] must be {N}")
        bias_ptr, bias_dt = bias.data_ptr(), _DT[bias.dtype]
    with torch.cuda.device(D.device):
        check(LIB.ac4k_linear_nvfp4(D.data_ptr(), _DT[D.dtype], A.data_ptr(), A_sf.data_ptr(),
                                    A_global_scale.data_ptr(), B.data_ptr(), B_sf.data_ptr(),
                                    B_global_scale.data_ptr(), bias_ptr, bias_dt, M, N, K, layout,
                                    _stream(D)),
              "linear_nvfp4")


def linear_nvfp4_gather(dst_ptrs, ldd, col_off, D_local, A, A_sf, A_global_scale, B, B_sf, B_global_scale, bias):
    """The GEMM of `linear_nvfp4` storing every tile to several [M, ldd] buffers at columns
    [col_off, col_off + N): the all-gather of the column-parallel layer fused into the epilogue
    (no counterpart in the reference).  `dst_ptrs`: device addresses of the destinations, this GPU's
    own buffer first; `D_local`: this GPU's buffer as a [M, ldd] tensor (for dtype, device, stream).
    N is taken from B."""
    _require(D_local.dim() == 2 and D_local.is_cuda and D_local.is_contiguous(), "d must be a contiguous 2d matrix")
    _require(D_local.dtype in (torch.bfloat16, torch.float16), "d must be bfloat16 or half")
    M = D_local.size(0)
    _require(D_local.size(1) == ldd, "ldd must be the row length of d")
    _check_tensor(A, torch.uint8, "a")
    _check_tensor(B, torch.uint8, "b")
    _require(A.dim() == 2 and B.dim() == 2 and A.size(0) == M and A.size(1) == B.size(1), "a / b shapes do not match")
    N, K = B.size(0), A.size(1) * 2
    kt = _ceil_div(K, 64)
    _check_tensor(A_sf, torch.float8_e4m3fn, "scale_a")
    _check_tensor(B_sf, torch.float8_e4m3fn, "scale_b")
    if A_sf.dim() == 3:
        layout = SF_AC4K
        _require(list(A_sf.shape) == [kt, _align_up(M, 16), 4], "scale_a has an invalid shape")
        _require(list(B_sf.shape) == [kt, _align_up(N, 16), 4], "scale_b has an invalid shape")
    else:
        layout = SF_TILE128X4
        _require(list(A_sf.shape) == [_ceil_div(M, 128), kt, 32, 4, 4], "scale_a has an invalid shape")
        _require(list(B_sf.shape) == [_ceil_div(N, 128), kt, 32, 4, 4], "scale_b has an invalid shape")
    _check_tensor(A_global_scale, torch.float32, "global_scale_a")
    _check_tensor(B_global_scale, torch.float32, "global_scale_b")
    bias_ptr, bias_dt = None, 0
    if bias is not None:
        _require(bias.dtype in _DT and bias.is_cuda and bias.is_contiguous(), "bias must be a contiguous cuda tensor")
        _require(bias.dim() == 2 and bias.size(0) == 1 and bias.size(1) == N, f"bias must be [1, {N}]")
        bias_ptr, bias_dt = bias.data_ptr(), _DT[bias.dtype]
    arr = (ctypes.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
    with torch.cuda.device(D_local.device):
        check(LIB.ac4k_linear_nvfp4_gather(arr, len(dst_ptrs), int(ldd), int(col_off), _DT[D_local.dtype],
                                           A.data_ptr(), A_sf.data_ptr(), A_global_scale.data_ptr(),
                                           B.data_ptr(), B_sf.data_ptr(), B_global_scale.data_ptr(),
                                           bias_ptr, bias_dt, M, N, K, layout, _stream(D_local)),
              "linear_nvfp4_gather")


def linear_nvfp4_requant(out, out_sf, out_global_scale, A, A_sf, A_global_scale, B, B_sf, B_global_scale, bias):
    """NVFP4 GEMM whose epilogue quantises the bf16 result to NVFP4 with the given global scale
    (no counterpart in the reference's linear path).  `out`: [M, N/2] uint8, `out_sf`: e4m3 scales in
    either layout (3-d [N/64, align16(M), 4] or 5-d [ceil(M/128), N/64, 32, 4, 4])."""
    _check_tensor(out, torch.uint8, "out")
    _require(out.dim() == 2, "out must be a 2d matrix")
    M, N = out.size(0), out.size(1) * 2
    _check_tensor(A, torch.uint8, "a")
    _check_tensor(B, torch.uint8, "b")
    _require(A.dim() == 2 and B.dim() == 2 and A.size(0) == M and B.size(0) == N and A.size(1) == B.size(1),
             "a / b / out shapes do not match")
    K = A.size(1) * 2
    kt = _ceil_div(K, 64)
    for t, nm in ((A_sf, "scale_a"), (B_sf, "scale_b"), (out_sf, "out_sf")):
        _check_tensor(t, torch.float8_e4m3fn, nm)
    if A_sf.dim() == 3:
        layout = SF_AC4K
        _require(list(A_sf.shape) == [kt, _align_up(M, 16), 4], "scale_a has an invalid shape")
        _require(list(B_sf.shape) == [kt, _align_up(N, 16), 4], "scale_b has an invalid shape")
    else:
        layout = SF_TILE128X4
        _require(list(A_sf.shape) == [_ceil_div(M, 128), kt, 32, 4, 4], "scale_a has an invalid shape")
        _require(list(B_sf.shape) == [_ceil_div(N, 128), kt, 32, 4, 4], "scale_b has an invalid shape")
    _require(N % 64 == 0, "N must be a multiple of 64")
    if out_sf.dim() == 3:
        out_layout = SF_AC4K
        _require(list(out_sf.shape) == [N // 64, _align_up(M, 16), 4], "out_sf has an invalid shape")
    else:
        out_layout = SF_TILE128X4
        _require(list(out_sf.shape) == [_ceil_div(M, 128), N // 64, 32, 4, 4], "out_sf has an invalid shape")
    for t, nm in ((A_global_scale, "global_scale_a"), (B_global_scale, "global_scale_b"), (out_global_scale, "out_global_scale")):
        _check_tensor(t, torch.float32, nm)
        _require(t.dim() == 0, f"{nm} must be a scalar")
    bias_ptr, bias_dt = None, 0
    if bias is not None:
        _require(bias.dtype in _DT and bias.is_cuda and bias.is_contiguous(), "bias must be a contiguous cuda tensor")
        _require(bias.dim() == 2 and bias.size(0) == 1 and bias.size(1) == N, f"bias must be [1, {N}]")
        bias_ptr, bias_dt = bias.data_ptr(), _DT[bias.dtype]
    with torch.cuda.device(out.device):
        check(LIB.ac4k_linear_nvfp4_requant(out.data_ptr(), out_sf.data_ptr(), out_global_scale.data_ptr(), out_layout,
                                            A.data_ptr(), A_sf.data_ptr(), A_global_scale.data_ptr(),
                                            B.data_ptr(), B_sf.data_ptr(), B_global_scale.data_ptr(),
                                            bias_ptr, bias_dt, M, N, K, layout, _stream(out)),
              "linear_nvfp4_requant")


def global_scale_bf16(out, input, max_scale):
    """out[()] = max|input| / max_scale on the device; stands in for the reference's Triton
    amax kernel (python/ac4k_kernel/ops/quant.py:21-59)."""
    _check_tensor(input, torch.bfloat16, "in")
    _check_tensor(out, torch.float32, "out")
    _require(out.dim() == 0, "out must be a scalar")
    with torch.cuda.device(input.device):
        check(LIB.ac4k_global_scale_bf16(input.data_ptr(), input.numel(), float(max_scale),
                                         out.data_ptr(), _stream(input)),
              "global_scale_bf16")


def mha_nvfp4_fwd(o, q, q_sf, q_global_scale, k, k_sf, k_global_scale, v, v_sf, v_global_scale, sm_scale):
    """o = softmax(sm_scale * q k^T) v on NVFP4 operands (ops.h:13-17; checks of
    lib/cuda/sm120/mha_nvfp4.cu:897-1010).  q: [B, H, Nq, Dqk/2], k: [B, H, Nkv, Dqk/2],
    v: [B, H, Dv, align64(Nkv)/2] (quantised along the keys, swizzle=True), o: bf16 [B, H, Nq, Dv] in any
    strides (the reference passes a permuted [B, N, H, D] buffer).  Block scales either in the reference's layout
    [B, H, K/64, align16(rows), 4] or tiled [B, H, ceil(rows/128), K/64, 32, 4, 4] (all three alike)."""
    _check_tensor(q, torch.uint8, "Q")
    _require(q.dim() == 4, "Q must be a 4D tensor")
    B, H, Nq = q.size(0), q.size(1), q.size(2)
    Dqk = q.size(3) * 2
    _require(Dqk % 16 == 0, "Dqk must be multiple of 16")
    _require(Dqk <= 128, "Dqk must be less than 128")
    _check_tensor(k, torch.uint8, "K")
    _require(k.dim() == 4, "K must be a 4D tensor")
    _require(k.size(0) == B, "K must have the same batch size as Q")
    _require(k.size(1) == H, "K must have the same head number as Q")
    Nkv = k.size(2)
    _require(k.size(3) == q.size(3), "K must have the same dim as Q")
    _check_tensor(v, torch.uint8, "V")
    _require(v.dim() == 4, "V must be a 4D tensor")
    _require(v.size(0) == B, "V must have the same batch size as Q")
    _require(v.size(1) == H, "V must have the same head number as Q")
    Dv = v.size(2)
    _require(v.size(3) * 2 == _align_up(Nkv, 64), "V must have the same sequence length as K")
    _require(Dv <= 128, "Dv must be less than 128")
    layout = SF_TILE128X4 if q_sf.dim() == 7 else SF_AC4K
    for name, sf, rows, red in (("q_sf", q_sf, Nq, Dqk), ("k_sf", k_sf, Nkv, Dqk), ("v_sf", v_sf, Dv, Nkv)):
        _check_tensor(sf, torch.float8_e4m3fn, name)
        if layout == SF_AC4K:       # the reference's layout and checks (mha_nvfp4.cu:915-1008)
            _require(sf.dim() == 5, f"{name} must be a 5D tensor")
            _require(list(sf.shape) == [B, H, _ceil_div(red, 64), _align_up(rows, 16), 4],
                     f"Meet invalid {name} shape {list(sf.shape)}")
        else:
            _require(sf.dim() == 7, f"{name} must be a 7D tensor like q_sf (tiled layout)")
            _require(list(sf.shape) == [B, H, _ceil_div(rows, 128), _ceil_div(red, 64), 32, 4, 4],
                     f"Meet invalid {name} shape {list(sf.shape)}")
    for name, g in (("q_global_scale", q_global_scale), ("k_global_scale", k_global_scale),
                    ("v_global_scale", v_global_scale)):
        _check_tensor(g, torch.float32, name)
        _require(g.dim() == 0, f"{name} must be a scalar")
    _require(isinstance(o, torch.Tensor) and o.is_cuda, "O must be a CUDA tensor")
    _require(o.dtype == torch.bfloat16, "O must be a bfloat16 tensor")
    _require(o.dim() == 4, "O must be a 4D tensor")
    _require(list(o.shape) == [B, H, Nq, Dv], f"O must have shape {[B, H, Nq, Dv]} but see {list(o.shape)}")
    with torch.cuda.device(o.device):
        check(LIB.ac4k_mha_nvfp4_fwd(o.data_ptr(), _I64x4(*o.stride()), q.data_ptr(), q_sf.data_ptr(),
                                     q_global_scale.data_ptr(), k.data_ptr(), k_sf.data_ptr(),
                                     k_global_scale.data_ptr(), v.data_ptr(), v_sf.data_ptr(),
                                     v_global_scale.data_ptr(), B, H, Nq, Nkv, Dqk, Dv, float(sm_scale),
                                     layout, _stream(o)),
              "mha_nvfp4_fwd")


def rope3d(x, grid_sizes, freqs, output):
    """3-D rotary position embedding (ops.h:50-54; checks of lib/cuda/sm120/rope3d.cu:133-165).
    x, output: bf16 [B, S, N, D]; grid_sizes: int32 [B, 3]; freqs: complex128 [max_pos, D // 2]."""
    _check_tensor(x, torch.bfloat16, "x")
    _check_tensor(grid_sizes, torch.int32, "grid_sizes")
    _check_tensor(freqs, torch.complex128, "freqs")
    _check_tensor(output, torch.bfloat16, "output")
    _require(x.dim() == 4, "x must be 4D tensor")
    _require(grid_sizes.dim() == 2, "grid_sizes must be 2D tensor")
    _require(freqs.dim() == 2, "freqs must be 2D tensor")
    _require(output.dim() == 4, "output must be 4D tensor")
    B, S, N, D = x.shape
    _require(grid_sizes.size(0) == B, "grid_sizes batch size must match x")
    _require(grid_sizes.size(1) == 3, "grid_sizes must have 3 dimensions (F, H, W)")
    _require(list(output.shape) == [B, S, N, D], "output shape must match x")
    _require(D % 2 == 0, "feature dimension must be even")
    _require(freqs.size(1) == D // 2, "freqs must have D / 2 columns")
    with torch.cuda.device(x.device):
        check(LIB.ac4k_rope3d(output.data_ptr(), x.data_ptr(), grid_sizes.data_ptr(), freqs.data_ptr(), B, S, N, D,
                              freqs.size(0), _stream(x)),
              "rope3d")


def mha_int8_x_fp8_fwd(o, q, q_sf, q_quantize_block_size, k, k_sf, k_quantize_block_size, v, v_sf, sm_scale):
    """o = softmax(sm_scale * q k^T) v with INT8 q, k and FP8 p, v (ops.h:19-25; checks of
    lib/cuda/sm120/mha_int8_x_fp8.cu:983-1060).  q: int8 [B, H, Nq, Dqk], q_sf: fp32 [B, H, ceil(Nq / q_block)];
    k: int8 [B, H, Nkv, Dqk], k_sf: fp32 [B, H, ceil(Nkv / k_block)]; v: e4m3 [B, H, Dv, align16(Nkv)] (quantised along
    the keys, swizzle=True, max_scale 2.25), v_sf: fp32 [B, H, align16(Dv)]; o: bf16 [B, H, Nq, Dv] in any strides."""
    _check_tensor(q, torch.int8, "Q")
    _require(q.dim() == 4, "Q must be a 4D tensor")
    B, H, Nq, Dqk = q.shape
    _require(Dqk % 16 == 0, "Dqk must be multiple of 16")
    _require(Dqk <= 128, "Dqk must be less than 128")
    qb, kb = int(q_quantize_block_size), int(k_quantize_block_size)
    _check_tensor(q_sf, torch.float32, "Q_SF")
    _require(q_sf.dim() == 3, "Q_SF must be a 3D tensor")
    _require(list(q_sf.shape) == [B, H, _ceil_div(Nq, qb)], f"Meet invalid Q_SF shape {list(q_sf.shape)}")
    _check_tensor(k, torch.int8, "K")
    _require(k.dim() == 4, "K must be a 4D tensor")
    _require(k.size(0) == B, "K must have the same batch size as Q")
    _require(k.size(1) == H, "K must have the same head number as Q")
    Nkv = k.size(2)
    _require(k.size(3) == Dqk, "K must have the same dim as Q")
    _check_tensor(k_sf, torch.float32, "K_SF")
    _require(k_sf.dim() == 3, "K_SF must be a 3D tensor")
    _require(list(k_sf.shape) == [B, H, _ceil_div(Nkv, kb)], f"Meet invalid K_SF shape {list(k_sf.shape)}")
    _check_tensor(v, torch.float8_e4m3fn, "V")
    _require(v.dim() == 4, "V must be a 4D tensor")
    _require(v.size(0) == B, "V must have the same batch size as Q")
    _require(v.size(1) == H, "V must have the same head number as Q")
    Dv = v.size(2)
    _require(v.size(3) == _align_up(Nkv, 16), "V must have the same sequence length as K")
    _require(Dv <= 128, "Dv must be less than 128")
    _check_tensor(v_sf, torch.float32, "V_SF")
    _require(v_sf.dim() == 3, "V_SF must be a 3D tensor")
    _require(list(v_sf.shape) == [B, H, _align_up(Dv, 16)], f"Meet invalid v_sf shape {list(v_sf.shape)}")
    _require(isinstance(o, torch.Tensor) and o.is_cuda, "O must be a CUDA tensor")
    _require(o.dtype == torch.bfloat16, "O must be a bfloat16 tensor")
    _require(o.dim() == 4, "O must be a 4D tensor")
    _require(list(o.shape) == [B, H, Nq, Dv], f"O must have shape {[B, H, Nq, Dv]} but see {list(o.shape)}")
    with torch.cuda.device(o.device):
        check(LIB.ac4k_mha_int8_x_fp8_fwd(o.data_ptr(), _I64x4(*o.stride()), q.data_ptr(), q_sf.data_ptr(), qb,
                                          k.data_ptr(), k_sf.data_ptr(), kb, v.data_ptr(), v_sf.data_ptr(), B, H, Nq,
                                          Nkv, Dqk, Dv, float(sm_scale), _stream(o)),
              "mha_int8_x_fp8_fwd")


def quantize_int8_block(out, scale, input, layout, block_size, sub=None):
    """INT8 quantisation in blocks of `block_size` tokens (all features of a head share the block's scale); stands in
    for the reference's Triton kernel (python/ac4k_kernel/ops/attention.py:18-99).  input: bf16 [B, N, H, D] ("BNHD")
    or [B, H, N, D] ("BHND"), any strides; out: int8 [B, H, N, align16(D)]; scale: fp32 [B, H, ceil(N / block_size)].
    sub: None, or a bf16 tensor of input's layout with one token ([B, 1, H, D] / [B, H, 1, D]): input - sub (a bf16 tensor
    subtraction) is quantised, without that tensor being written."""
    _require(layout in ("BNHD", "BHND"), f"Unsupported layout: {layout}")
    _require(isinstance(input, torch.Tensor) and input.is_cuda and input.dtype == torch.bfloat16 and input.dim() == 4,
             "in must be a 4D bfloat16 CUDA tensor")
    x = input.permute(0, 2, 1, 3) if layout == "BNHD" else input
    B, H, N, D = x.shape
    _check_tensor(out, torch.int8, "out")
    _check_tensor(scale, torch.float32, "scale")
    _require(list(out.shape) == [B, H, N, _align_up(D, 16)], "out has an invalid shape")
    _require(list(scale.shape) == [B, H, _ceil_div(N, int(block_size))], "scale has an invalid shape")
    sub_ptr, sub_strides = None, None
    if sub is not None:
        u = sub.permute(0, 2, 1, 3) if layout == "BNHD" else sub
        _require(u.is_cuda and u.dtype == torch.bfloat16 and list(u.shape) == [B, H, 1, D] and u.stride(3) == 1,
                 "sub must be a bfloat16 CUDA tensor with one token and contiguous features")
        sub_ptr, sub_strides = u.data_ptr(), (ctypes.c_int64 * 2)(u.stride(0), u.stride(1))
    with torch.cuda.device(input.device):
        check(LIB.ac4k_quantize_int8_block(out.data_ptr(), scale.data_ptr(), x.data_ptr(), _I64x4(B, H, N, D),
                                           _I64x4(*x.stride()), int(block_size), sub_ptr, sub_strides, _stream(input)),
              "quantize_int8_block")
