"""GPU parity tests of the NVFP4 GEMM: CUDA path (through the C ABI, via the reference-shaped
`quantize` / `linear` wrappers) vs the restatement in oracle/.

Tolerance (stated by the target this build follows): relative L2 <= 2e-3 against
cast(alpha * dequant(A) @ dequant(B)^T + bias), and per element at most 2 ulps of the output
dtype.  The products of e2m1 values and e4m3 scales are exact in fp32, so the only error
sources are the accumulation order and the final rounding; the oracle accumulates in fp64.
Where an output suffers cancellation (|out| far below the magnitude of its partial sums) an
ulp of the *result* is not a meaningful yardstick, so the per-element bound also allows
2^-22 of sum_k |a_k b_k| (a few fp32 roundings of the largest partial sum).
"""
import os
import random

import numpy as np
import pytest
import torch

from oracle import emulation as emu
from tests.helpers import bf16_from_bits, gaussian

pytestmark = pytest.mark.gpu

ULP_REL = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -23}


@pytest.fixture(scope="module")
def ops():
    from ac4k_kernel_b200 import ops as o
    return o


def gemm_reference(a4, asf, ag, b4, bsf, bg, bias, out_dtype, device):
    """fp64-accumulated oracle and the magnitude sum_k |a_k b_k| * alpha, on `device`."""
    to = lambda t: t.to(device)
    ad = emu.dequantize_nvfp4_ref(to(a4), to(asf), None).double()
    bd = emu.dequantize_nvfp4_ref(to(b4), to(bsf), None).double()
    alpha = (to(ag).float() * to(bg).float()).double()
    acc = ad @ bd.t() * alpha
    mag = ad.abs() @ bd.abs().t() * alpha
    if bias is not None:
        acc = acc + to(bias).reshape(1, -1).double()
        mag = mag + to(bias).reshape(1, -1).double().abs()
    return acc, mag


def assert_gemm_close(out, acc64, mag64, out_dtype):
    ref = acc64.to(out_dtype)
    o = out.double()
    r = ref.double()
    assert not bool(torch.isnan(o).any()), "NaN in output"
    rel = float((o - r).norm() / r.norm().clamp(min=1e-300))
    assert rel <= 2e-3, f"relative L2 {rel}"
    # ulp of the output dtype at |ref|
    e = torch.frexp(r.abs().clamp(min=1e-300))[1] - 1
    ulp = torch.ldexp(torch.ones_like(r), e) * ULP_REL[out_dtype]
    tol = 2 * ulp + mag64 * 2.0 ** -22
    bad = (o - r).abs() > tol
    assert not bool(bad.any()), f"{int(bad.sum())} of {bad.numel()} elements off by more than 2 ulps"
    # the strict reading of the target (2 ulps of the result, no allowance for cancelled sums): how many
    # elements need the allowance, and the worst error in ulps of the result
    err_ulp = (o - r).abs() / ulp
    strict_bad = int((err_ulp > 2).sum())
    return rel, float(err_ulp.max()), strict_bad


STRICT_LOG = []     # (case, elements, elements beyond a strict 2-ulp bound, worst strict-ulp error)


def run_case(ops, m, n, k, seed=0, layout="ac4k", bias_dtype=None, out_dtype=None, a=None, b=None,
             oracle_device="cpu", strict_name=None, strict_frac=None):
    a = gaussian((m, k), seed=seed) if a is None else a
    b = gaussian((n, k), seed=seed + 1) if b is None else b
    ad, bd = a.cuda(), b.cuda()
    a4, asf, ag = ops.quantize(ad, 0, 1, sf_layout=layout)
    b4, bsf, bg = ops.quantize(bd, 0, 1, sf_layout=layout)
    bias = None
    if bias_dtype is not None:
        bias = gaussian((1, n), seed=seed + 2).to(bias_dtype).cuda()
    out = None
    if out_dtype is not None:
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    res = ops.linear(a4, asf, ag, b4, bsf, bg, bias=bias, out=out)
    torch.cuda.synchronize()
    from ac4k_kernel_b200 import _lib
    assert _lib.device_status() == 0
    odt = torch.bfloat16 if out_dtype is None else out_dtype
    assert res.dtype == odt and tuple(res.shape) == (m, n)
    acc, mag = gemm_reference(a4, asf, ag, b4, bsf, bg, bias, odt, oracle_device)
    rel, worst, strict_bad = assert_gemm_close(res.to(oracle_device), acc, mag, odt)
    if strict_name is not None:
        STRICT_LOG.append((strict_name, m * n, strict_bad, worst))
        print(f"[strict 2-ulp] {strict_name}: {strict_bad} of {m * n} elements beyond 2 ulps of the result "
              f"({strict_bad / (m * n):.2e}), worst {worst:.2f} ulps, relative L2 {rel:.2e}")
        if strict_frac is not None:
            # only outputs that suffer cancellation (|out| far below its partial sums) may need the allowance
            assert strict_bad <= strict_frac * m * n, (strict_name, strict_bad, m * n)
    return rel, worst


@pytest.mark.parametrize("layout", ["ac4k", "128x4"])
def test_config1(ops, layout):
    """BASELINE config 1: A [128,512], B [256,512], N(0,1), seed 0; operands bit-exact, GEMM in tolerance."""
    g = torch.Generator().manual_seed(0)
    A = torch.randn((128, 512), generator=g).bfloat16()
    B = torch.randn((256, 512), generator=g).bfloat16()
    a4, asf, ag = ops.quantize(A.cuda(), 0, 1, sf_layout=layout)
    ra4, rasf, rag = emu.quantize_nvfp4_ref(A, sf_layout=layout)
    assert torch.equal(a4.cpu(), ra4) and torch.equal(asf.view(torch.uint8).cpu(), rasf.view(torch.uint8))
    assert torch.equal(ag.cpu(), rag)
    run_case(ops, 128, 256, 512, layout=layout, a=A, b=B)


# the reference's own shape list (test/test_linear_bench.py:167-177)
REF_SHAPES = [(128, 128, 128), (10, 512, 512), (1024, 1024, 384), (130, 384, 256), (666, 768, 512),
              (123, 321, 256), (10, 15, 512), (1, 4, 256), (64, 64, 128), (12, 23, 55)]


@pytest.mark.parametrize("layout", ["ac4k", "128x4"])
@pytest.mark.parametrize("shape", REF_SHAPES)
def test_reference_shapes(ops, shape, layout):
    run_case(ops, *shape, seed=9567, layout=layout)


@pytest.mark.parametrize("m,n,k,odt,bdt", [
    (12, 23, 5, torch.float32, None),
    (1, 2, 50, torch.float16, torch.bfloat16), (1, 2, 50, torch.float16, torch.float16),
    (2, 3, 51, torch.float16, torch.float32), (3, 2, 50, torch.bfloat16, torch.bfloat16),
    (4, 2, 50, torch.bfloat16, torch.float16), (5, 3, 51, torch.bfloat16, torch.float32),
    (1, 21, 50, torch.float32, torch.bfloat16), (1, 22, 50, torch.float32, torch.float16),
    (2, 33, 51, torch.float32, torch.float32),
    (200, 264, 320, torch.float16, torch.float32), (130, 136, 192, torch.float32, torch.bfloat16),
])
def test_bias_and_output_dtypes(ops, m, n, k, odt, bdt):
    """test/test_linear_bench.py:178-205 plus two tile-crossing shapes."""
    run_case(ops, m, n, k, seed=3, bias_dtype=bdt, out_dtype=odt)


@pytest.mark.parametrize("m,n,k", [(260, 392, 320), (262, 392, 320), (1028, 520, 1088), (1026, 520, 1088)])
@pytest.mark.parametrize("bdt", [None, torch.float32])
def test_row_layout_scale_paths(ops, m, n, k, bdt):
    """Scales in the reference's layout reach the CTA-pair kernel in two ways: with M and N multiples of 4 the
    operand rows are permuted by the loads and the scales are used as they lie in memory; otherwise warps re-order
    the scales.  Both against the restatement, ragged tiles in both directions."""
    run_case(ops, m, n, k, seed=31, layout="ac4k", bias_dtype=bdt, out_dtype=torch.bfloat16)


def test_random_shapes(ops):
    """test/test_linear_bench.py:156-161: 20 random M, N, K in [2, 555]."""
    rng = random.Random(9567)
    for i in range(20):
        m, n, k = rng.randint(2, 555), rng.randint(2, 555), rng.randint(2, 555)
        run_case(ops, m, n, k, seed=100 + i, layout="ac4k" if i % 2 else "128x4")


def test_bias_1d_and_default_output(ops):
    a = gaussian((40, 128), seed=1).cuda()
    b = gaussian((72, 128), seed=2).cuda()
    bias = gaussian((72,), seed=3).cuda()
    a4, asf, ag = ops.quantize(a, 0, 1)
    b4, bsf, bg = ops.quantize(b, 0, 1)
    out = ops.linear(a4, asf, ag, b4, bsf, bg, bias=bias)
    acc, mag = gemm_reference(a4, asf, ag, b4, bsf, bg, bias.reshape(1, -1), torch.bfloat16, "cuda")
    assert_gemm_close(out, acc, mag, torch.bfloat16)


def test_golden_reference_emulation(ops, golden_dir):
    """Outputs of the reference's get_torch_results (tests/golden/make_golden.py) vs the CUDA path,
    at the reference's own tolerance (test_linear_bench.py:152)."""
    z = np.load(os.path.join(golden_dir, "nvfp4_linear_reference_emulation.npz"))
    for i in range(int(z["n_cases"])):
        a = bf16_from_bits(z[f"l{i}_a"]).cuda()
        b = bf16_from_bits(z[f"l{i}_b"]).cuda()
        bias = None
        if f"l{i}_bias" in z:
            bias = torch.from_numpy(z[f"l{i}_bias"]).to(eval(str(z[f"l{i}_bias_dtype"]))).cuda()
        odt = eval(str(z[f"l{i}_out_dtype"]))
        a4, asf, ag = ops.quantize(a, 0, 1)
        b4, bsf, bg = ops.quantize(b, 0, 1)
        out = torch.empty((a.shape[0], b.shape[0]), dtype=odt, device="cuda")
        ops.linear(a4, asf, ag, b4, bsf, bg, bias=bias, out=out)
        ref = torch.from_numpy(z[f"l{i}_out"])
        torch.testing.assert_close(out.float().cpu(), ref, atol=1e-2, rtol=1e-2)
        assert float((out.float().cpu() - ref).norm() / ref.norm()) < 2e-3


def test_argument_checks(ops):
    a = gaussian((16, 64), seed=1).cuda()
    a4, asf, ag = ops.quantize(a, 0, 1)
    with pytest.raises(RuntimeError, match="B size"):
        ops.linear(a4, asf, ag, a4[:, :16].contiguous(), asf, ag)
    with pytest.raises(RuntimeError, match="bias shape"):
        ops.linear(a4, asf, ag, a4, asf, ag, bias=torch.zeros((1, 5), device="cuda"))
    with pytest.raises(RuntimeError, match="scalar"):
        ops.linear(a4, asf, ag.reshape(1), a4, asf, ag)


# ------------------------------------------------------------------ full-size configurations
def _outlier_activations(shape, seed, frac, mul):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, generator=g, device="cuda")
    mask = torch.rand(shape, generator=g, device="cuda") < frac
    return torch.where(mask, x * mul, x).bfloat16()


def _weights(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * 0.02).bfloat16()


@pytest.mark.parametrize("layout", ["ac4k", "128x4"])
def test_config2_full(ops, layout):
    """BASELINE config 2: 4096^3, activations N(0,1) with 0.5% x30 outliers, weights N(0,0.02)."""
    run_case(ops, 4096, 4096, 4096, layout=layout, oracle_device="cuda",
             a=_outlier_activations((4096, 4096), 0, 0.005, 30.0), b=_weights((4096, 4096), 1),
             strict_name=f"config 2 (4096^3, {layout})", strict_frac=1e-3)


@pytest.mark.parametrize("m", [1, 16, 64])
def test_config3_decode_shapes(ops, m):
    """BASELINE config 3: M in {1,16,64}, K = N = 8192."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((m, 8192), generator=g, device="cuda").bfloat16()
    for layout in ("128x4", "ac4k"):
        run_case(ops, m, 8192, 8192, layout=layout, oracle_device="cuda", a=x, b=_weights((8192, 8192), 1))


@pytest.mark.parametrize("m,n,k,odt,bdt", [
    # decode-shape kernel (M <= 64): K slices are the CTAs of a cluster, added through distributed shared memory
    (5, 2048, 4096, torch.bfloat16, torch.float32),     # 16 tiles, 16 stages -> 4 slices
    (33, 1024, 8192, torch.float16, torch.bfloat16),    # 8 tiles -> 4 slices, 64-row activation box (3-stage ring)
    (17, 16384, 2048, torch.bfloat16, None),            # 128 tiles -> 2 slices (4 would not fit one wave)
    (64, 8192, 1024, torch.float32, torch.float32),     # 4 stages only -> 1 slice
    (3, 4100, 2048, torch.bfloat16, None),              # ragged N (N % 128 != 0, odd tail tile)
    (1, 8200, 1088, torch.float16, None),               # K % 256 != 0: a short last stage in the last slice
    # single-CTA kernel (65 <= M <= 128): fp32 partial sums in scratch memory + reduction kernel
    (128, 512, 8192, torch.float32, None),              # 4 tiles -> 8 slices
    (100, 1024, 8192, torch.bfloat16, torch.bfloat16),  # 8 tiles -> 8 slices
    (96, 2304, 16384, torch.float16, None),             # 18 tiles -> 8 slices
    (128, 512, 4096, torch.float32, None),              # K too short to slice: one pass
])
def test_split_k_paths(ops, m, n, k, odt, bdt):
    """Few output tiles and a long K: the library slices K over more CTAs.  The shapes reach the plans named
    beside them through the library's own planning (no measurement switch is involved)."""
    run_case(ops, m, n, k, seed=21, layout="128x4", bias_dtype=bdt, out_dtype=odt, oracle_device="cuda")
    run_case(ops, m, n, k, seed=22, layout="ac4k", bias_dtype=bdt, out_dtype=odt, oracle_device="cuda")


def test_reference_8192_cube(ops):
    """test/test_linear_bench.py:174."""
    g = torch.Generator(device="cuda").manual_seed(9567)
    a = torch.randn((8192, 8192), generator=g, device="cuda").bfloat16()
    b = torch.randn((8192, 8192), generator=g, device="cuda").bfloat16()
    run_case(ops, 8192, 8192, 8192, oracle_device="cuda", a=a, b=b, strict_name="8192^3 (ac4k)", strict_frac=1e-3)


def test_config5_single_gpu_linearity(ops):
    """BASELINE config 5 at full size on one GPU: M=8192, K=8192, N=28672.  Besides the
    tolerance check, the column-parallel property the multi-GPU variant relies on: computing
    any N-shard alone gives bit-identical columns."""
    a = _outlier_activations((8192, 8192), 0, 0.005, 30.0)
    w = _weights((28672, 8192), 1)
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
    w4, wsf, wg = ops.quantize(w, 0, 1, sf_layout="128x4")
    out = ops.linear(a4, asf, ag, w4, wsf, wg)
    acc, mag = gemm_reference(a4, asf, ag, w4, wsf, wg, None, torch.bfloat16, "cuda")
    rel, worst, strict_bad = assert_gemm_close(out, acc, mag, torch.bfloat16)
    print(f"[strict 2-ulp] config 5 (8192 x 28672 x 8192, 128x4): {strict_bad} of {out.numel()} elements beyond 2 ulps "
          f"of the result ({strict_bad / out.numel():.2e}), worst {worst:.2f} ulps, relative L2 {rel:.2e}")
    assert strict_bad <= 1e-3 * out.numel()
    del acc, mag
    for world in (2, 8):
        ns = 28672 // world
        r = world - 1
        shard = ops.linear(a4, asf, ag, w4[r * ns:(r + 1) * ns], wsf[r * ns // 128:(r + 1) * ns // 128], wg)
        assert torch.equal(shard, out[:, r * ns:(r + 1) * ns])
    out2 = ops.linear(a4, asf, ag, w4, wsf, wg)
    assert torch.equal(out, out2)
    # the reference's scale layout gives the same bytes: both layouts hold the same scales
    a4r, asfr, agr = ops.quantize(a, 0, 1, sf_layout="ac4k")
    w4r, wsfr, wgr = ops.quantize(w, 0, 1, sf_layout="ac4k")
    out3 = ops.linear(a4r, asfr, agr, w4r, wsfr, wgr)
    assert torch.equal(out, out3)


def test_repeatable_under_requantisation(ops):
    """Forty runs of config 2, each after re-running the quantisers (which moves the kernel's
    timing around), must give bit-identical outputs: a race between the roles of the GEMM kernel
    shows up as a 32-row block that differs in a fraction of the runs."""
    a = _outlier_activations((4096, 4096), 0, 0.005, 30.0)
    w = _weights((4096, 4096), 1)
    first = None
    for it in range(40):
        a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
        w4, wsf, wg = ops.quantize(w, 0, 1, sf_layout="128x4")
        out = ops.linear(a4, asf, ag, w4, wsf, wg)
        if first is None:
            first = out.clone()
            acc, mag = gemm_reference(a4, asf, ag, w4, wsf, wg, None, torch.bfloat16, "cuda")
            assert_gemm_close(first, acc, mag, torch.bfloat16)
            del acc, mag
        else:
            assert torch.equal(out, first), f"run {it} differs from run 0"


@pytest.mark.parametrize("layout", ["ac4k", "128x4"])
@pytest.mark.parametrize("m,n,k,ldd,col_off,odt,with_bias,n_dst", [
    (512, 512, 1024, 1536, 512, torch.bfloat16, False, 3),
    (300, 264, 256, 800, 8, torch.bfloat16, True, 3),        # ragged tiles, 16-byte aligned rows only
    (128, 256, 512, 256, 0, torch.float16, False, 3),        # M of a single row tile, dense destination
    (1024, 512, 512, 4096, 3584, torch.bfloat16, False, 8),  # the largest number of destinations (an 8-GPU node), last column block
])
def test_gather_epilogue_on_one_gpu(ops, layout, m, n, k, ldd, col_off, odt, with_bias, n_dst):
    """The fused all-gather epilogue with all destinations on one GPU: n_dst [M, ldd] buffers get
    columns [col_off, col_off + N) equal to the plain GEMM's output; the other columns stay as
    they were."""
    from ac4k_kernel_b200 import _cuda_ops
    a = gaussian((m, k), seed=3).cuda()
    b = gaussian((n, k), seed=4).cuda()
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout=layout)
    b4, bsf, bg = ops.quantize(b, 0, 1, sf_layout=layout)
    bias = gaussian((1, n), seed=5).to(odt).cuda() if with_bias else None
    plain = torch.empty((m, n), dtype=odt, device="cuda")
    _cuda_ops.linear_nvfp4(plain, a4, asf, ag, b4, bsf, bg, bias)
    bufs = [torch.full((m, ldd), -7.0, dtype=odt, device="cuda") for _ in range(n_dst)]
    _cuda_ops.linear_nvfp4_gather([t.data_ptr() for t in bufs], ldd, col_off, bufs[0], a4, asf, ag, b4, bsf, bg, bias)
    torch.cuda.synchronize()
    for t in bufs:
        assert torch.equal(t[:, col_off:col_off + n], plain)
        assert bool((t[:, :col_off] == -7.0).all()) and bool((t[:, col_off + n:] == -7.0).all())


def test_gather_argument_checks(ops):
    from ac4k_kernel_b200 import _cuda_ops
    a = gaussian((256, 256), seed=3).cuda()
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
    buf = torch.zeros((256, 512), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):      # columns do not fit
        _cuda_ops.linear_nvfp4_gather([buf.data_ptr()], 512, 384, buf, a4, asf, ag, a4, asf, ag, None)
    with pytest.raises(RuntimeError):      # col_off not a multiple of 8
        _cuda_ops.linear_nvfp4_gather([buf.data_ptr()], 512, 4, buf, a4, asf, ag, a4, asf, ag, None)
    with pytest.raises(RuntimeError):      # too many destinations
        _cuda_ops.linear_nvfp4_gather([buf.data_ptr()] * 9, 512, 0, buf, a4, asf, ag, a4, asf, ag, None)


@pytest.mark.parametrize("in_layout,out_layout", [("128x4", "128x4"), ("128x4", "ac4k"), ("ac4k", "128x4")])
@pytest.mark.parametrize("m,n,k,with_bias", [
    (512, 512, 1024, False),
    (300, 320, 256, True),          # ragged row tile, N = 64 * 5
    (100, 192, 512, False),         # fewer rows than one tile
    (4096, 4096, 4096, False),      # config 2
])
def test_requant_epilogue_equals_linear_then_quantize(ops, in_layout, out_layout, m, n, k, with_bias):
    """linear_requant == quantize(linear(...) in bf16, given global scale), bit for bit: packed
    codes, block scales and their zero padding."""
    from ac4k_kernel_b200 import _cuda_ops
    from ac4k_kernel_b200.ops.utils import align_up, ceil_div
    a = gaussian((m, k), seed=21).cuda()
    b = (gaussian((n, k), seed=22) * 0.05).bfloat16().cuda()
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout=in_layout)
    b4, bsf, bg = ops.quantize(b, 0, 1, sf_layout=in_layout)
    bias = gaussian((1, n), seed=23).cuda() if with_bias else None
    y = ops.linear(a4, asf, ag, b4, bsf, bg, bias=bias)                    # bf16 [m, n]
    # the caller's calibrated output scale: here the true one, scaled so that some blocks saturate
    g_out = (y.float().abs().max() / (6.0 * 448.0) * 0.75).reshape(()).contiguous()
    ref4 = torch.empty((m, n // 2), dtype=torch.uint8, device="cuda")
    if out_layout == "ac4k":
        ref_sf = torch.empty((n // 64, align_up(m, 16), 4), dtype=torch.float8_e4m3fn, device="cuda")
    else:
        ref_sf = torch.empty((ceil_div(m, 128), n // 64, 32, 4, 4), dtype=torch.float8_e4m3fn, device="cuda")
    _cuda_ops.quantize_nvfp4(ref4, ref_sf, y, g_out, 0, 1, False)
    out4, out_sf, _ = ops.linear_requant(a4, asf, ag, b4, bsf, bg, g_out, bias=bias, sf_layout=out_layout)
    torch.cuda.synchronize()
    assert torch.equal(out4, ref4)
    assert torch.equal(out_sf.view(torch.uint8), ref_sf.view(torch.uint8))
    # and the fused output feeds the next layer like the two-call output does
    w2 = (gaussian((256, n), seed=24) * 0.05).bfloat16().cuda()
    w24, w2sf, w2g = ops.quantize(w2, 0, 1, sf_layout=out_layout)
    z_ref = ops.linear(ref4, ref_sf, g_out, w24, w2sf, w2g)
    z = ops.linear(out4, out_sf, g_out, w24, w2sf, w2g)
    assert torch.equal(z, z_ref)


def test_requant_argument_checks(ops):
    a = gaussian((256, 256), seed=3).cuda()
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
    b = gaussian((96, 256), seed=4).cuda()              # N = 96 is not a multiple of 64
    b4, bsf, bg = ops.quantize(b, 0, 1, sf_layout="128x4")
    with pytest.raises(RuntimeError):
        ops.linear_requant(a4, asf, ag, b4, bsf, bg, ag)


@pytest.mark.parametrize("layout", ["ac4k", "128x4"])
@pytest.mark.parametrize("m,n,k,bdt", [
    (129, 136, 64, None),              # pair kernel, one K step, one ragged tile in both directions
    (257, 264, 576, torch.float32),    # 9 K steps: full stage of 8 + ragged stage of 1; two row tiles
    (512, 136, 1088, None),            # 17 K steps, narrow ragged N
    (300, 520, 4160, torch.bfloat16),  # 65 K steps (8 full stages + 1), three column tiles
    (2048, 2048, 2048, None),          # whole tiles, more tiles than clusters
])
def test_pair_kernel_edges(ops, layout, m, n, k, bdt):
    """Shapes that take the CTA-pair kernel (M, N > 128, N % 8 == 0) at its edges: ragged last
    pipeline stage, ragged tiles, a single K step."""
    run_case(ops, m, n, k, seed=31, layout=layout, bias_dtype=bdt, oracle_device="cuda")


def test_graph_capture_and_two_streams(ops):
    """The calls are asynchronous on the caller's stream and capturable: a CUDA graph of
    quantize + linear replays to the eager result, and two streams running different problems
    at the same time (one of them on the split-K path) do not disturb each other."""
    from ac4k_kernel_b200 import _lib
    a = gaussian((512, 1024), seed=41).cuda()
    b = gaussian((768, 1024), seed=42).cuda()
    b4, bsf, bg = ops.quantize(b, 0, 1, sf_layout="128x4")
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
    eager = ops.linear(a4, asf, ag, b4, bsf, bg)
    out = torch.empty_like(eager)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        with torch.cuda.graph(g, stream=st):
            qa, qsf, qg = ops.quantize(a, 0, 1, sf_layout="128x4")
            ops.linear(qa, qsf, qg, b4, bsf, bg, out=out)
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
    # two streams
    a2 = gaussian((16, 4096), seed=43).cuda()
    b2 = gaussian((2048, 4096), seed=44).cuda()
    a24, a2sf, a2g = ops.quantize(a2, 0, 1, sf_layout="ac4k")
    b24, b2sf, b2g = ops.quantize(b2, 0, 1, sf_layout="ac4k")
    ref2 = ops.linear(a24, a2sf, a2g, b24, b2sf, b2g)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs1, outs2 = [], []
    for _ in range(10):
        with torch.cuda.stream(s1):
            outs1.append(ops.linear(a4, asf, ag, b4, bsf, bg))
        with torch.cuda.stream(s2):
            outs2.append(ops.linear(a24, a2sf, a2g, b24, b2sf, b2g))
    torch.cuda.synchronize()
    assert all(torch.equal(o, eager) for o in outs1)
    assert all(torch.equal(o, ref2) for o in outs2)
    assert _lib.device_status() == 0
