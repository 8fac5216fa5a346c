"""CPU/torch restatement of ac4k_kernel's NVFP4 linear path.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA kernels: it is imported by the tests, by the
smoke check and by the CPU-baseline leg of the benchmark, never by the product package.
Every function works on CPU tensors and (because it only uses elementwise fp32 torch ops,
which are IEEE round-to-nearest on both devices) on CUDA tensors as well, so full-size
inputs can be checked on the GPU against the same arithmetic.

Parity status: PINNED.  The reference ships no golden files, but its own test oracles
(`test/test_quantize_bench.py` `get_ref` / `qunatize_fp8`, `test/test_linear_bench.py`
`get_torch_results`) were executed on CPU against this restatement; their outputs on seeded
inputs are stored under tests/golden/ (see tests/golden/make_golden.py).

Reference lines followed (paths inside the ac4k_kernel project):
  * global scale            python/ac4k_kernel/ops/quant.py:21-59,198-200
  * NVFP4 quantiser math    lib/cuda/sm120/quantize_nvfp4.cu:73,113-147  (order of fp32 ops)
  * NVFP4 layouts, padding  lib/cuda/sm120/quantize_nvfp4.cu:56-70,83,107-108,150-155;
                            test/test_quantize_bench.py:29-83
  * K permutation "swizzle" lib/cuda/sm120/quantize_nvfp4.cu:86-100; test_quantize_bench.py:60-64
  * nibble order / LUT      lib/cuda/common/math.cuh:62-85; test/test_linear_bench.py:15-50
  * dequantise + matmul     test/test_linear_bench.py:53-107; lib/cuda/sm120/linear_nvfp4.cu:586-633
  * per-token FP8           lib/cuda/sm120/quantize_fp8.cu:91-176; test_quantize_bench.py:256-300
  * per-token INT8          lib/cuda/sm120/quantize_int8.cu:55-59,125-165
  * 128x4 scale tile        test/utils.py:15-23

The reference kernels use `rcp.approx.ftz` and `--use_fast_math`; this restatement (and the
CUDA kernels checked against it) use correctly rounded fp32 operations in the same order, so
that CPU, GPU-torch and the hand-written kernels agree bit for bit.  How far that is from the
reference's kernels themselves is measured, not assumed: its quantiser and RoPE kernels are built
for sm_100a by oracle/build_ref.py and run beside the CUDA path in
tests/test_reference_kernels_gpu.py (RoPE and, for global scales with an exactly rounded
approximate reciprocal, the NVFP4 quantiser: every byte equal).
"""
from __future__ import annotations

import torch

BLOCK = 16            # elements per scale block            (quant.py:190)
PACK_SF = 4           # scales packed per 32-bit word       (quant.py:192)
CROSS_ALIGN = 16      # scale rows are padded to 16         (quant.py:193)
REDUCE_ALIGN = 64     # K is padded to 64                   (quant.py:194)
E2M1_MAX = 6.0
E4M3_MAX = 448.0
ONE_SIXTH = 0.16666667163372040   # fp32(1/6), the literal in quantize_nvfp4.cu:126

E2M1_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
               -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def ceil_div(a, b):
    return (a + b - 1) // b


def align_up(a, b):
    return ceil_div(a, b) * b


# ----------------------------------------------------------------------------------------
# scalar format conversions
# ----------------------------------------------------------------------------------------
def e4m3_rne_sat_bits(s: torch.Tensor) -> torch.Tensor:
    """fp32 (>= 0 or NaN) -> e4m3fn byte, round-to-nearest-even, saturating to 448.

    Written with integer/fp32 arithmetic only (no torch fp8 cast) so that it can be checked
    against torch's own cast.  NaN maps to 0x7F like `cvt.rn.satfinite.e4m3x2.f32`.
    """
    s = s.to(torch.float32)
    nan = torch.isnan(s)
    neg = torch.signbit(s)
    a = s.abs().clamp(max=E4M3_MAX)
    a = torch.where(nan, torch.zeros_like(a), a)
    # quantum of the e4m3 grid around a: 2^(e-3) for normals (e >= -6), 2^-9 below 2^-6
    ad = a.double()
    e = (torch.frexp(ad)[1] - 1).clamp(min=-6).double()     # floor(log2(a)), exact
    q = torch.ldexp(torch.ones_like(ad), (e - 3.0).to(torch.int32))
    n = torch.round(ad / q)                  # torch.round is half-to-even; a/q exact in fp64
    v = n * q                                # value on the grid (may carry into next binade)
    # encode v
    ve = (torch.frexp(v)[1] - 1).clamp(min=-6).double()
    mant = v / torch.ldexp(torch.ones_like(v), ve.to(torch.int32))
    is_sub = v < 2.0 ** -6
    exp_field = torch.where(is_sub, torch.zeros_like(ve), ve + 7.0)
    man_field = torch.where(is_sub, v / 2.0 ** -9, (mant - 1.0) * 8.0)
    bits = (exp_field * 8.0 + man_field).to(torch.int64)
    bits = torch.where(v == 0, torch.zeros_like(bits), bits)
    bits = bits | (neg.to(torch.int64) << 7)
    bits = torch.where(nan, torch.full_like(bits, 0x7F), bits)
    return bits.to(torch.uint8)


def e4m3_bits_to_float(b: torch.Tensor) -> torch.Tensor:
    return b.contiguous().view(torch.float8_e4m3fn).to(torch.float32)


def e2m1_rne_sat_codes(y: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit e2m1 code (0..15), RNE, saturate to +-6, sign of zero kept.

    Ties go to the code with an even mantissa bit: 0.25->0, 0.75->1, 1.25->1, 1.75->2,
    2.5->2, 3.5->4, 5->4.  NaN -> 0x7 (what `cvt.rn.satfinite.e2m1x2.f32` returns).
    """
    y = y.to(torch.float32)
    a = y.abs()
    code = torch.zeros(y.shape, dtype=torch.uint8, device=y.device)
    code = torch.where(a > 0.25, torch.full_like(code, 1), code)
    code = torch.where(a >= 0.75, torch.full_like(code, 2), code)
    code = torch.where(a > 1.25, torch.full_like(code, 3), code)
    code = torch.where(a >= 1.75, torch.full_like(code, 4), code)
    code = torch.where(a > 2.5, torch.full_like(code, 5), code)
    code = torch.where(a >= 3.5, torch.full_like(code, 6), code)
    code = torch.where(a > 5.0, torch.full_like(code, 7), code)
    code = code | (torch.signbit(y).to(torch.uint8) << 3)
    code = torch.where(torch.isnan(y), torch.full_like(code, 7), code)
    return code


def e2m1_codes_to_float(code: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=code.device)
    return lut[code.long()]


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    """[..., n] bytes -> [..., 2n] codes; element 2j is the LOW nibble of byte j
    (test_linear_bench.py:39-49)."""
    lo = packed & 0x0F
    hi = (packed >> 4) & 0x0F
    return torch.stack((lo, hi), dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def pack_fp4(codes: torch.Tensor) -> torch.Tensor:
    c = codes.reshape(*codes.shape[:-1], codes.shape[-1] // 2, 2)
    return (c[..., 0] | (c[..., 1] << 4)).to(torch.uint8)


# ----------------------------------------------------------------------------------------
# layout helpers
# ----------------------------------------------------------------------------------------
def _canonical(x: torch.Tensor, cross_dim: int, reduce_dim: int):
    """Permute to [others..., cross, reduce] and flatten the others into one batch dim."""
    nd = x.ndim
    assert 2 <= nd <= 4
    if cross_dim < 0:
        cross_dim += nd
    if reduce_dim < 0:
        reduce_dim += nd
    assert cross_dim != reduce_dim
    others = [i for i in range(nd) if i not in (cross_dim, reduce_dim)]
    lead = [x.shape[i] for i in others]
    xp = x.permute(*others, cross_dim, reduce_dim).contiguous()
    m, k = x.shape[cross_dim], x.shape[reduce_dim]
    return xp.reshape(-1, m, k), lead, m, k


def sf_ac4k_to_rows(sf: torch.Tensor, m: int, nblk: int) -> torch.Tensor:
    """[KT, M16, 4] -> [m, nblk]: one scale per (row, 16-block) (test_linear_bench.py:7-12)."""
    t = sf.permute(1, 0, 2)
    return t.reshape(t.shape[0], -1)[:m, :nblk]


def sf_rows_to_ac4k(rows: torch.Tensor, m16: int, kt: int) -> torch.Tensor:
    """[m, nblk] (any 1-byte dtype) -> [KT, M16, 4], zero filled padding."""
    m, nblk = rows.shape
    full = torch.zeros((m16, kt * 4), dtype=rows.dtype, device=rows.device)
    full[:m, :nblk] = rows
    return full.reshape(m16, kt, 4).permute(1, 0, 2).contiguous()


def sf_rows_to_tile128x4(rows: torch.Tensor, kt: int) -> torch.Tensor:
    """[m, nblk] bytes -> [ceil(m/128), KT, 32, 4, 4]; byte (r, b) lands at
    tile (r/128, b/4), offset (r%32)*16 + ((r%128)/32)*4 + b%4 (test/utils.py:15-23)."""
    m, nblk = rows.shape
    mt = ceil_div(m, 128)
    full = torch.zeros((mt * 128, kt * 4), dtype=rows.dtype, device=rows.device)
    full[:m, :nblk] = rows
    t = full.reshape(mt, 4, 32, kt, 4)          # (mt, r/32, r%32, kt, b%4)
    return t.permute(0, 3, 2, 1, 4).contiguous()  # (mt, kt, r%32, r/32, b%4)


def sf_tile128x4_to_rows(sf: torch.Tensor, m: int, nblk: int) -> torch.Tensor:
    mt, kt = sf.shape[0], sf.shape[1]
    t = sf.permute(0, 3, 2, 1, 4).reshape(mt * 128, kt * 4)
    return t[:m, :nblk]


def permute_k_nvfp4(x: torch.Tensor) -> torch.Tensor:
    """K permutation used for attention's V ("swizzle"): every 32 elements are viewed as
    [4, 4, 2] and transposed to [4(b), 4(a), 2] (test_quantize_bench.py:60-64)."""
    s = x.shape
    return x.reshape(-1, 4, 4, 2).permute(0, 2, 1, 3).reshape(s)


def permute_k_fp8(x: torch.Tensor) -> torch.Tensor:
    """FP8 variant: every 16 elements viewed as [2, 4, 2] -> [4, 2, 2]
    (test_quantize_bench.py:276-280)."""
    s = x.shape
    return x.reshape(-1, 2, 4, 2).permute(0, 2, 1, 3).reshape(s)


# ----------------------------------------------------------------------------------------
# NVFP4 quantiser
# ----------------------------------------------------------------------------------------
def global_scale_ref(x: torch.Tensor, max_scale: float = E2M1_MAX * E4M3_MAX) -> torch.Tensor:
    """0-dim fp32: max|x| / max_scale (quant.py:49-59; test_quantize_bench.py:19-20)."""
    amax = x.abs().amax().to(torch.float32) if x.numel() else torch.zeros((), device=x.device)
    return amax / torch.tensor(max_scale, dtype=torch.float32, device=x.device)


def quantize_nvfp4_ref(x: torch.Tensor, cross_dim: int = 0, reduce_dim: int = 1,
                       global_scale: torch.Tensor | None = None, swizzle: bool = False,
                       sf_layout: str = "ac4k", max_scale: float = E2M1_MAX * E4M3_MAX):
    """bf16 -> (packed u8 [..., M, Kp/2], scales e4m3, global scale fp32 0-dim).

    Arithmetic order (all fp32, round to nearest, no fused multiply-add):
        alpha = 1 / g                       (0 when g == 0)
        s     = alpha * (amax_block * fp32(1/6));  sf = e4m3_rne_sat(s)
        r     = sf == 0 ? 0 : alpha * (1 / float(sf))
        code  = e2m1_rne_sat(float(x) * r)
    """
    assert x.dtype == torch.bfloat16
    g = global_scale_ref(x, max_scale) if global_scale is None else global_scale.to(torch.float32)
    xb, lead, m, k = _canonical(x, cross_dim, reduce_dim)
    kp = align_up(k, REDUCE_ALIGN)
    nb = xb.shape[0]
    xf = torch.zeros((nb, m, kp), dtype=torch.float32, device=x.device)
    xf[:, :, :k] = xb.to(torch.float32)
    if swizzle:
        xf = permute_k_nvfp4(xf)
    one = torch.ones((), dtype=torch.float32, device=x.device)
    alpha = torch.where(g == 0, torch.zeros_like(g), one / g)
    blocks = xf.reshape(nb, m, kp // BLOCK, BLOCK)
    amax_b = blocks.abs().amax(dim=-1)
    s = alpha * (amax_b * torch.tensor(ONE_SIXTH, dtype=torch.float32, device=x.device))
    sf_bits = e4m3_rne_sat_bits(s)
    sf_f = e4m3_bits_to_float(sf_bits)
    r = torch.where(sf_f == 0, torch.zeros_like(sf_f), alpha * (one / sf_f))
    codes = e2m1_rne_sat_codes(blocks * r.unsqueeze(-1)).reshape(nb, m, kp)
    packed = pack_fp4(codes).reshape(*lead, m, kp // 2)
    kt = kp // REDUCE_ALIGN
    if sf_layout == "ac4k":
        m16 = align_up(m, CROSS_ALIGN)
        sf = torch.stack([sf_rows_to_ac4k(sf_bits[i], m16, kt) for i in range(nb)])
        sf = sf.reshape(*lead, kt, m16, 4)
    elif sf_layout == "128x4":
        sf = torch.stack([sf_rows_to_tile128x4(sf_bits[i], kt) for i in range(nb)])
        sf = sf.reshape(*lead, ceil_div(m, 128), kt, 32, 4, 4)
    else:
        raise ValueError(sf_layout)
    return packed, sf.view(torch.float8_e4m3fn), g


def dequantize_nvfp4_ref(packed: torch.Tensor, sf: torch.Tensor, g: torch.Tensor | None,
                         sf_layout: str | None = None) -> torch.Tensor:
    """2-D packed [rows, Kp/2] + scales -> fp32 [rows, Kp]; value = e2m1 * e4m3 (* g)
    (test_linear_bench.py:53-67 with global_scale passed as 1/g there)."""
    rows, kp2 = packed.shape
    kp = kp2 * 2
    if sf_layout is None:
        sf_layout = "ac4k" if sf.dim() == 3 else "128x4"
    sfb = sf.view(torch.uint8)
    if sf_layout == "ac4k":
        sr = sf_ac4k_to_rows(sfb, rows, kp // BLOCK)
    else:
        sr = sf_tile128x4_to_rows(sfb, rows, kp // BLOCK)
    vals = e2m1_codes_to_float(unpack_fp4(packed)).reshape(rows, kp // BLOCK, BLOCK)
    out = (vals * e4m3_bits_to_float(sr).unsqueeze(-1)).reshape(rows, kp)
    if g is not None:
        out = out * g.to(torch.float32)
    return out


def linear_nvfp4_ref(a, a_sf, a_g, b, b_sf, b_g, bias=None, out_dtype=torch.bfloat16,
                     accum_dtype=torch.float32):
    """out = cast(alpha * dequant(A) @ dequant(B)^T + bias), alpha = a_g * b_g in fp32
    (linear_nvfp4.cu:586-633; test_linear_bench.py:70-107).  `accum_dtype=torch.float64`
    gives the exact-accumulation variant used to bound kernel error."""
    ad = dequantize_nvfp4_ref(a, a_sf, None).to(accum_dtype)
    bd = dequantize_nvfp4_ref(b, b_sf, None).to(accum_dtype)
    acc = ad @ bd.t()
    alpha = (a_g.to(torch.float32) * b_g.to(torch.float32)).to(accum_dtype)
    acc = acc * alpha
    if bias is not None:
        acc = acc + bias.reshape(1, -1).to(accum_dtype)
    return acc.to(out_dtype)


# ----------------------------------------------------------------------------------------
# per-token FP8 / INT8 quantisers
# ----------------------------------------------------------------------------------------
def _rowwise_common(x, cross_dim, reduce_dim, scale_max: float, permute):
    assert x.dtype == torch.bfloat16
    xb, lead, m, k = _canonical(x, cross_dim, reduce_dim)
    kp = align_up(k, 16)
    m16 = align_up(m, CROSS_ALIGN)
    nb = xb.shape[0]
    xf = torch.zeros((nb, m, kp), dtype=torch.float32, device=x.device)
    xf[:, :, :k] = xb.to(torch.float32)
    if permute:
        xf = permute_k_fp8(xf)
    smax = torch.tensor(float(scale_max), dtype=torch.float32, device=x.device)
    amax = xf.abs().amax(dim=-1)                           # [nb, m]
    sf = torch.zeros((nb, m16), dtype=torch.float32, device=x.device)
    sf[:, :m] = amax / smax                                # quantize_fp8.cu:124
    recip = smax / amax                                    # quantize_fp8.cu:132 (inf for a zero row)
    y = xf * recip.unsqueeze(-1)                           # 0 * inf = NaN, as in the reference
    return y, sf.reshape(*lead, m16), lead, m, kp


def quantize_fp8_ref(x, cross_dim=0, reduce_dim=1, scale_max: float = 448.0, swizzle=False):
    """Per-row e4m3: returns (e4m3 [..., M, align16(K)], fp32 scales [..., align16(M)])."""
    y, sf, lead, m, kp = _rowwise_common(x, cross_dim, reduce_dim, scale_max, swizzle)
    # satfinite: +-448 clamp keeps the sign, NaN -> 0x7F
    bits = e4m3_rne_sat_bits(y)
    return bits.reshape(*lead, m, kp).view(torch.float8_e4m3fn), sf


def quantize_int8_ref(x, cross_dim=0, reduce_dim=1, scale_max: int = 127):
    """Per-row int8 with `cvt.rni.sat.s8.f32`: round half to even, clamp [-128, 127], NaN -> 0."""
    y, sf, lead, m, kp = _rowwise_common(x, cross_dim, reduce_dim, float(int(scale_max)), False)
    q = torch.round(y).clamp(-128, 127)
    q = torch.where(torch.isnan(y), torch.zeros_like(q), q)
    return q.to(torch.int8).reshape(*lead, m, kp), sf


# ----------------------------------------------------------------------------------------
# NVFP4 attention
# ----------------------------------------------------------------------------------------
P_GLOBAL_RCP = 2688.0     # 6 * 448: reciprocal of the fixed global scale of P (mha_nvfp4.cu:253)
LOG2E = 1.4426950408889634


def _quantize_p_tile(p: torch.Tensor):
    """[rows, 128] fp32 probabilities (already in the stored key order) -> their NVFP4 values as fp32,
    still divided by the global scale: e2m1 * e4m3 per block of 16 (mha_nvfp4.cu:246-319: block scale
    e4m3(2688 * (max / 6)), elements scaled by 2688 / scale)."""
    rows = p.shape[0]
    blk = p.reshape(rows, -1, BLOCK)
    one_sixth = torch.tensor(ONE_SIXTH, dtype=torch.float32, device=p.device)
    g = torch.tensor(P_GLOBAL_RCP, dtype=torch.float32, device=p.device)
    sfb = e4m3_rne_sat_bits(g * (blk.amax(dim=-1) * one_sixth))
    sff = e4m3_bits_to_float(sfb)
    scale = torch.where(sff == 0, torch.zeros_like(sff), g / sff)
    codes = e2m1_rne_sat_codes(blk * scale.unsqueeze(-1))
    return (e2m1_codes_to_float(codes) * sff.unsqueeze(-1)).reshape(rows, -1)


def mha_nvfp4_ref(q, q_sf, q_g, k, k_sf, k_g, v, v_sf, v_g, sm_scale: float, nkv: int,
                  tile: int = 128, out_dtype=torch.bfloat16):
    """softmax(sm_scale * Q K^T) V on quantised operands, walking the keys in tiles of `tile` with a running
    maximum and sum the way the attention kernels do (lib/cuda/sm120/mha_nvfp4.cu:640-760 per key tile:
    S, row max, P = exp(S - max) in fp32, l += sum(P), P re-quantised to NVFP4, O = O * exp(max_old - max)
    + P V; :860-893: O * v_g / (2688 * l)).
      q: [B, H, Nq, Dp/2], k: [B, H, Nkv, Dp/2], v: [B, H, Dv, align64(Nkv)/2] packed, V's keys in the
      permuted order of `quantize(v, 3, N_dim, swizzle=True)`; scales in either layout; nkv = true key count.
    Returns [B, H, Nq, Dv]."""
    B, H, nq = q.shape[0], q.shape[1], q.shape[2]
    dv = v.shape[2]
    kvp = v.shape[3] * 2
    dev = q.device
    c1 = (q_g.to(torch.float32) * k_g.to(torch.float32) * torch.tensor(sm_scale, dtype=torch.float32, device=dev)
          * torch.tensor(LOG2E, dtype=torch.float32, device=dev))
    # stored position -> key index inside every group of 32 (inverse view of permute_k_nvfp4)
    pos = torch.arange(kvp, device=dev)
    key_of_pos = permute_k_nvfp4(pos.to(torch.float32)).to(torch.long)
    out = torch.empty((B, H, nq, dv), dtype=out_dtype, device=dev)
    layout = "ac4k" if q_sf.dim() == 5 else "128x4"
    for b in range(B):
        for h in range(H):
            qd = dequantize_nvfp4_ref(q[b, h], q_sf[b, h], None, layout)
            kd = dequantize_nvfp4_ref(k[b, h], k_sf[b, h], None, layout)
            vd = dequantize_nvfp4_ref(v[b, h], v_sf[b, h], None, layout)          # [Dv, kvp], permuted keys
            s_all = qd @ kd.t()                                                    # [Nq, Nkv] before the scales
            m = torch.full((nq,), float("-inf"), dtype=torch.float32, device=dev)
            l = torch.zeros((nq,), dtype=torch.float32, device=dev)
            o = torch.zeros((nq, dv), dtype=torch.float32, device=dev)
            for j0 in range(0, nkv, tile):
                j1 = min(j0 + tile, nkv)
                s = s_all[:, j0:j1]
                m_new = torch.maximum(m, s.amax(dim=1) * c1)
                p = torch.exp2(s * c1 - m_new.unsqueeze(1))
                a = torch.exp2(m - m_new)
                l = l * a + p.sum(dim=1)
                # P in the stored key order of this tile, zero where the key does not exist
                width = min(tile, kvp - j0)
                pf = torch.zeros((nq, width), dtype=torch.float32, device=dev)
                keys = key_of_pos[j0:j0 + width]
                valid = keys < nkv
                pf[:, valid] = p[:, keys[valid] - j0]
                pq = _quantize_p_tile(pf)
                o = o * a.unsqueeze(1) + pq @ vd[:, j0:j0 + width].t()
                m = m_new
            res = o * (v_g.to(torch.float32) / (torch.tensor(P_GLOBAL_RCP, device=dev) * l)).unsqueeze(1)
            out[b, h] = res.to(out_dtype)
    return out


def attention_nvfp4_ref(q, k, v, layout: str = "BNHD", sf_layout: str = "128x4"):
    """The reference's `attention(..., precision="nvfp4")` (python/ac4k_kernel/ops/attention.py:102-138) on this
    module's quantiser: q, k quantised along the head dimension, v along the keys with the K permutation."""
    n_dim = 1 if layout == "BNHD" else 2
    nkv = k.shape[n_dim]
    qq, qs, qg = quantize_nvfp4_ref(q, n_dim, 3, sf_layout=sf_layout)
    kq, ks, kg = quantize_nvfp4_ref(k, n_dim, 3, sf_layout=sf_layout)
    vq, vs, vg = quantize_nvfp4_ref(v, 3, n_dim, swizzle=True, sf_layout=sf_layout)
    o = mha_nvfp4_ref(qq, qs, qg, kq, ks, kg, vq, vs, vg, 1.0 / (q.shape[-1] ** 0.5), nkv)
    return o.permute(0, 2, 1, 3).contiguous() if layout == "BNHD" else o


# ----------------------------------------------------------------------------------------
# 3-D rotary position embedding
# ----------------------------------------------------------------------------------------
def rope_params_ref(max_pos: int, dim: int, theta: float = 10000.0) -> torch.Tensor:
    """complex128 [max_pos, dim // 2]: exp(i * p * theta^(-2c / dim)) (test/test_rope_3d_apply.py:5-12)."""
    assert dim % 2 == 0
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64),
                          torch.arange(0, dim, 2, dtype=torch.float64) / dim)
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv)
    return torch.polar(torch.ones_like(ang), ang)


def rope3d_ref(x: torch.Tensor, grid_sizes: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x bf16 [B, S, N, D], grid_sizes int [B, 3] = (F, H, W), freqs complex128 [max_pos, D // 2] -> bf16 [B, S, N, D].

    Position s < F * H * W sits at (f, h, w) = (s // (H W), (s % (H W)) // W, s % W); of the C = D // 2 complex pairs of
    every head the first C - 2 (C // 3) are multiplied by freqs[f, c], the next C // 3 by freqs[h, c], the last C // 3 by
    freqs[w, c]; products in complex128, result -> fp32 -> bf16.  Positions behind the grid are copied from x
    (test/test_rope_3d_apply.py:14-42; the kernel, lib/cuda/sm120/rope3d.cu:44-129, does the same arithmetic per
    element and leaves those positions unwritten)."""
    B, S, N, D = x.shape
    C = D // 2
    c2 = C // 3
    c1 = C - 2 * c2
    out = x.clone()
    col = torch.arange(C, device=x.device)
    for b in range(B):
        F_, H_, W_ = (int(v) for v in grid_sizes[b].tolist())
        n = min(F_ * H_ * W_, S)
        if n == 0:
            continue
        s = torch.arange(n, device=x.device)
        f, h, w = s // (H_ * W_), (s % (H_ * W_)) // W_, s % W_
        row = torch.where(col[None, :] < c1, f[:, None], torch.where(col[None, :] < c1 + c2, h[:, None], w[:, None]))
        fac = freqs[row, col[None, :].expand(n, C)]                       # [n, C] complex128
        xc = torch.view_as_complex(x[b, :n].to(torch.float64).reshape(n, N, C, 2))
        y = torch.view_as_real(xc * fac[:, None, :]).reshape(n, N, D)
        out[b, :n] = y.to(torch.float32).to(torch.bfloat16)
    return out


# ----------------------------------------------------------------------------------------
# INT8 x FP8 attention
# ----------------------------------------------------------------------------------------
EXP_OFFSET = 7.5          # log2 units taken off the row maximum so that P uses e4m3's range (mha_int8_x_fp8.cu:119-121)
V_SCALE_MAX = 2.25        # largest |V| after its per-channel FP8 quantisation (mha_int8_x_fp8.cu:119; attention.py:171-176)


def quantize_int8_block_ref(x: torch.Tensor, layout: str, block: int):
    """bf16 [B, N, H, D] ("BNHD") or [B, H, N, D] ("BHND") -> (int8 [B, H, N, align16(D)], fp32 [B, H, ceil(N / block)]).
    One scale per `block` consecutive tokens of a head: max|x| / 127; values trunc(x / scale), 0 for an all-zero block
    (python/ac4k_kernel/ops/attention.py:18-48: `tl.cast` to int8 truncates toward zero; :51-99 shapes).  The division
    is a true fp32 division here and in the CUDA kernel; Triton's may differ in the last bit."""
    assert x.dtype == torch.bfloat16 and x.dim() == 4
    xb = x.permute(0, 2, 1, 3) if layout == "BNHD" else x
    B, H, N, D = xb.shape
    nblk = ceil_div(N, block)
    xf = torch.zeros((B, H, nblk * block, D), dtype=torch.float32, device=x.device)
    xf[:, :, :N] = xb.to(torch.float32)
    blk = xf.reshape(B, H, nblk, block * D)
    scale = blk.abs().amax(dim=-1) / torch.tensor(127.0, dtype=torch.float32, device=x.device)
    q = torch.where(scale.unsqueeze(-1) == 0, torch.zeros_like(blk), torch.trunc(blk / scale.unsqueeze(-1)))
    y = torch.zeros((B, H, N, align_up(D, 16)), dtype=torch.int8, device=x.device)
    y[..., :D] = q.reshape(B, H, nblk * block, D)[:, :, :N].to(torch.int8)
    return y, scale


def mha_int8_x_fp8_ref(q, q_sf, q_block: int, k, k_sf, k_block: int, v, v_sf, sm_scale: float, tile: int = 128,
                       fp16_tile_accumulate: bool = False, out_dtype=torch.bfloat16):
    """softmax(sm_scale * Q K^T) V on INT8 q, k and FP8 p, v, walking the keys in tiles of `tile` the way the kernels do
    (lib/cuda/sm120/mha_int8_x_fp8.cu:640-700 scores, :700-715 maximum with the 7.5 offset, :717-790 P and the row sum,
    :795-880 P V, :893-910 the final scaling).
      q: int8 [B, H, Nq, Dp], q_sf: fp32 [B, H, ceil(Nq / q_block)]; k: int8 [B, H, Nkv, Dp], k_sf likewise with k_block;
      v: e4m3 [B, H, Dv, align16(Nkv)] with the keys in the order of `quantize(v, 3, N_dim, swizzle=True,
      precision="fp8e4m3")`, v_sf: fp32 [B, H, align16(Dv)].
    `fp16_tile_accumulate` rounds every tile's P V to fp16 before it is added to O, as the reference's MMA does; the
    tcgen05 kernel accumulates in fp32.  Returns [B, H, Nq, Dv]."""
    B, H, nq, _ = q.shape
    nkv, dv, kvp = k.shape[2], v.shape[2], v.shape[3]
    dev = q.device
    f32 = lambda t: torch.tensor(t, dtype=torch.float32, device=dev)
    c0 = f32(sm_scale) * f32(LOG2E)
    key_of_pos = permute_k_fp8(torch.arange(kvp, device=dev).to(torch.float32)).to(torch.long)
    out = torch.empty((B, H, nq, dv), dtype=out_dtype, device=dev)
    rows = torch.arange(nq, device=dev)
    for b in range(B):
        for h in range(H):
            s_int = (q[b, h].to(torch.float64) @ k[b, h].to(torch.float64).t()).to(torch.float32)   # exact: |S| < 2^24
            c_row = c0 * q_sf[b, h][rows // q_block]                                                # [Nq]
            vnat = torch.zeros((dv, kvp), dtype=torch.float32, device=dev)
            vnat[:, key_of_pos] = v[b, h].to(torch.float32)                                         # natural key order
            m = torch.full((nq,), float("-inf"), dtype=torch.float32, device=dev)
            l = torch.zeros((nq,), dtype=torch.float32, device=dev)
            o = torch.zeros((nq, dv), dtype=torch.float32, device=dev)
            for j0 in range(0, nkv, tile):
                j1 = min(j0 + tile, nkv)
                cols = torch.arange(j0, j1, device=dev)
                c = c_row[:, None] * k_sf[b, h][cols // k_block][None, :]
                s = s_int[:, j0:j1] * c
                m_new = torch.maximum(m, s.amax(dim=1) - EXP_OFFSET)
                p = torch.exp2(s - m_new[:, None])
                a = torch.exp2(m - m_new)
                l = l * a + p.sum(dim=1)
                p8 = e4m3_bits_to_float(e4m3_rne_sat_bits(p))
                pv = p8 @ vnat[:, j0:j1].t()
                if fp16_tile_accumulate:
                    pv = pv.to(torch.float16).to(torch.float32)
                o = o * a[:, None] + pv
                m = m_new
            out[b, h] = (o * (v_sf[b, h][:dv][None, :] / l[:, None])).to(out_dtype)
    return out


def attention_int8_x_fp8_ref(q, k, v, layout: str = "BNHD", q_block: int = 64, k_block: int = 128):
    """The reference's `attention(..., precision="int8+fp8e4m3")` (python/ac4k_kernel/ops/attention.py:141-193) on this
    module's quantisers."""
    n_dim = 1 if layout == "BNHD" else 2
    k = k - k.mean(dim=n_dim, keepdim=True)
    qq, qs = quantize_int8_block_ref(q, layout, q_block)
    kq, ks = quantize_int8_block_ref(k, layout, k_block)
    vq, vs = quantize_fp8_ref(v, 3, n_dim, V_SCALE_MAX, swizzle=True)
    o = mha_int8_x_fp8_ref(qq, qs, q_block, kq, ks, k_block, vq, vs, 1.0 / (q.shape[-1] ** 0.5))
    return o.permute(0, 2, 1, 3).contiguous() if layout == "BNHD" else o
