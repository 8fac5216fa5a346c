"""GPU parity tests of the quantisers: CUDA path (through the C ABI) vs the restatement in
oracle/, bit-exact on packed bytes, scale bytes and global scale."""
import os

import numpy as np
import pytest
import torch

from oracle import emulation as emu
from tests.helpers import bf16_from_bits, gaussian

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from ac4k_kernel_b200 import ops as o
    return o


def _check_nvfp4(ops, x_cpu, cd=0, rd=1, swizzle=False, layout="ac4k", oracle_device="cpu"):
    x = x_cpu.cuda()
    out, sf, g = ops.quantize(x, cd, rd, swizzle=swizzle, sf_layout=layout)
    torch.cuda.synchronize()
    xo = x if oracle_device == "cuda" else x_cpu
    ro, rsf, rg = emu.quantize_nvfp4_ref(xo, cd, rd, swizzle=swizzle, sf_layout=layout)
    assert out.shape == ro.shape and sf.shape == rsf.shape
    assert torch.equal(g.cpu(), rg.cpu()), (float(g), float(rg))
    assert torch.equal(sf.view(torch.uint8).cpu(), rsf.view(torch.uint8).cpu()), "scale bytes differ"
    neq = (out.cpu() != ro.cpu())
    assert not bool(neq.any()), f"{int(neq.sum())} packed bytes differ"
    return out, sf, g


@pytest.mark.parametrize("layout", ["ac4k", "128x4"])
def test_config1_bit_exact(ops, layout):
    _check_nvfp4(ops, gaussian((128, 512), seed=0), layout=layout)
    _check_nvfp4(ops, gaussian((256, 512), seed=1), layout=layout)


@pytest.mark.parametrize("layout", ["ac4k", "128x4"])
@pytest.mark.parametrize("shape", [(1, 64), (7, 8), (130, 384), (123, 320), (10, 520), (555, 1000),
                                   (16, 8192), (1, 8192), (300, 24)])
def test_ragged_contiguous(ops, shape, layout):
    _check_nvfp4(ops, gaussian(shape, seed=sum(shape), outlier_frac=0.01, outlier_mul=50.0), layout=layout)


@pytest.mark.parametrize("layout", ["ac4k", "128x4"])
@pytest.mark.parametrize("shape,cd,rd,sw", [
    ((12, 55), 0, 1, False),       # K not a multiple of 8 -> strided kernel
    ((96, 80), 1, 0, False),       # transposed read
    ((37, 200), 0, 1, True),       # K permutation
    ((50, 33), 1, 0, True),
    ((3, 20, 70), 1, 2, False),
    ((2, 3, 40, 24), 3, 1, True),
    ((2, 70, 5, 32), 1, 3, False),  # attention-style q/k
    ((2, 3, 64, 128), 2, 3, False),  # batched contiguous rows -> tiled kernel with outer dims
])
def test_strided_and_permuted(ops, shape, cd, rd, sw, layout):
    _check_nvfp4(ops, gaussian(shape, seed=7), cd, rd, sw, layout)


@pytest.mark.parametrize("layout", ["ac4k", "128x4"])
@pytest.mark.parametrize("sw", [False, True])
@pytest.mark.parametrize("shape,cd,rd", [
    ((300, 130), 1, 0),            # rows contiguous, K strided: the transposing kernel, ragged in both directions
    ((64, 2), 1, 0),               # two rows
    ((2, 200, 3, 96), 3, 1),       # attention's V: [B, N, H, D] reduced over the keys
    ((1, 1000, 2, 128), 3, 1),
    ((1, 129, 1, 256), 3, 1),      # two row tiles, K one past a tile
])
def test_contiguous_rows_strided_k(ops, shape, cd, rd, sw, layout):
    _check_nvfp4(ops, gaussian(shape, seed=11, outlier_frac=0.01, outlier_mul=30.0), cd, rd, sw, layout)


def test_golden_known_answers_through_cuda(ops, golden_dir):
    """The reference's known-answer construction ({+-1,+-2,+-4,+-6} inputs, get_ref outputs)."""
    z = np.load(os.path.join(golden_dir, "nvfp4_quantize_known_answer.npz"))
    for i in range(int(z["n_cases"])):
        x = bf16_from_bits(z[f"q{i}_in"]).cuda()
        cd, rd, sw = (int(v) for v in z[f"q{i}_meta"])
        out, sf, g = ops.quantize(x, cd, rd, swizzle=bool(sw))
        deq = emu.e2m1_codes_to_float(emu.unpack_fp4(out.cpu()))
        np.testing.assert_allclose(deq.numpy(), z[f"q{i}_deq_codes"], atol=1e-3, rtol=1e-6)
        np.testing.assert_array_equal(sf.view(torch.uint8).cpu().numpy(), z[f"q{i}_sf"])
        np.testing.assert_allclose(g.cpu().numpy(), z[f"q{i}_g"], rtol=1e-6)


def test_zero_tensor_zero_blocks_negative_zero(ops):
    x = torch.zeros((32, 128), dtype=torch.bfloat16)
    _check_nvfp4(ops, x)
    x[3, 5] = 2.0
    x[4, 17] = -0.0
    x[9, 64:80] = -1e-30
    out, sf, g = _check_nvfp4(ops, x)
    codes = emu.unpack_fp4(out.cpu())
    assert codes[4, 17] == 8 and codes[3, 5] == 7


def test_outputs_fully_written(ops):
    """Callers allocate with torch.empty: every byte of out and sf, padding included, must be
    written (quantize_nvfp4.cu:83,107-108,150-155)."""
    x = gaussian((17, 72), seed=5).cuda()
    for layout, sf_shape in (("ac4k", (2, 32, 4)), ("128x4", (1, 2, 32, 4, 4))):
        out = torch.full((17, 64), 0xAB, dtype=torch.uint8, device="cuda")
        sf = torch.full(sf_shape, 0x55, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
        o2, s2, g = ops.quantize(x, 0, 1, output=out, sf=sf)
        ro, rsf, _ = emu.quantize_nvfp4_ref(x.cpu(), sf_layout=layout)
        assert torch.equal(out.cpu(), ro) and torch.equal(sf.view(torch.uint8).cpu(), rsf.view(torch.uint8))


def test_global_scale_odd_sizes_and_alignment(ops):
    from ac4k_kernel_b200.ops.quant import _global_scale
    base = gaussian((100003,), seed=11).cuda()
    for off, n in [(0, 100003), (1, 99999), (3, 5), (5, 1), (7, 4099), (0, 8)]:
        x = base[off:off + n]
        g = _global_scale(x, 2688.0)
        assert torch.equal(g.cpu(), emu.global_scale_ref(x.cpu()))


def test_full_size_config4_nvfp4(ops):
    """BASELINE config 4 at full size, checked on the GPU against the same arithmetic in torch,
    plus a CPU check of a row subset."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((32768, 8192), generator=g, device="cuda")
    mask = torch.rand((32768, 8192), generator=g, device="cuda") < 0.01
    x = torch.where(mask, x * 50.0, x).bfloat16()
    del mask
    out, sf, gs = ops.quantize(x, 0, 1)
    out2, sf2, _ = ops.quantize(x, 0, 1, sf_layout="128x4")
    assert torch.equal(out, out2)
    assert torch.equal(gs.cpu(), emu.global_scale_ref(x).cpu())
    rows_sf = emu.sf_ac4k_to_rows(sf.view(torch.uint8), 32768, 512)
    rows_sf2 = emu.sf_tile128x4_to_rows(sf2.view(torch.uint8), 32768, 512)
    assert torch.equal(rows_sf, rows_sf2)
    for r0 in range(0, 32768, 4096):           # GPU-torch oracle in slabs to bound memory
        ro, rsf, _ = emu.quantize_nvfp4_ref(x[r0:r0 + 4096], global_scale=gs)
        assert torch.equal(out[r0:r0 + 4096], ro)
        assert torch.equal(rows_sf[r0:r0 + 4096], emu.sf_ac4k_to_rows(rsf.view(torch.uint8), 4096, 512))
    idx = torch.arange(0, 32768, 997)
    ro, rsf, _ = emu.quantize_nvfp4_ref(x[idx.cuda()].cpu(), global_scale=gs.cpu())
    assert torch.equal(out[idx.cuda()].cpu(), ro)
    # run-to-run determinism
    out3, sf3, _ = ops.quantize(x, 0, 1)
    assert torch.equal(out, out3) and torch.equal(sf.view(torch.uint8), sf3.view(torch.uint8))


# ---------------------------------------------------------------------------- FP8 / INT8
def _check_rowwise(ops, x_cpu, precision, cd=0, rd=1, swizzle=False, max_scale=None, device="cpu"):
    x = x_cpu.cuda()
    out, sf = ops.quantize(x, cd, rd, precision=precision, swizzle=swizzle, max_scale=max_scale)
    xo = x if device == "cuda" else x_cpu
    if precision == "fp8e4m3":
        ro, rsf = emu.quantize_fp8_ref(xo, cd, rd, 448.0 if max_scale is None else max_scale, swizzle)
        a, b = out.view(torch.uint8).cpu(), ro.view(torch.uint8).cpu()
    else:
        ro, rsf = emu.quantize_int8_ref(xo, cd, rd, 127 if max_scale is None else max_scale)
        a, b = out.cpu(), ro.cpu()
    assert out.shape == ro.shape and sf.shape == rsf.shape
    assert torch.equal(sf.cpu(), rsf.cpu()), "row scales differ"
    assert torch.equal(a, b), f"{int((a != b).sum())} bytes differ"


@pytest.mark.parametrize("precision", ["fp8e4m3", "int8"])
@pytest.mark.parametrize("shape", [(64, 48), (100, 16), (17, 1024), (5, 1032), (33, 8192), (3, 20000),
                                   (7, 10), (1, 8)])
def test_rowwise_contiguous(ops, precision, shape):
    _check_rowwise(ops, gaussian(shape, seed=shape[1], outlier_frac=0.01, outlier_mul=50.0), precision)


@pytest.mark.parametrize("shape,cd,rd,sw", [((77, 79), 0, 1, True), ((2, 70, 5, 32), 3, 1, True),
                                            ((40, 24), 1, 0, False), ((3, 20, 70), 1, 2, False)])
def test_rowwise_strided(ops, shape, cd, rd, sw):
    _check_rowwise(ops, gaussian(shape, seed=9), "fp8e4m3", cd, rd, sw, max_scale=2.25)
    if not sw:
        _check_rowwise(ops, gaussian(shape, seed=9), "int8", cd, rd)


def test_fp8_golden_known_answers(ops, golden_dir):
    z = np.load(os.path.join(golden_dir, "fp8_quantize_known_answer.npz"))
    for i in range(int(z["n_cases"])):
        x = bf16_from_bits(z[f"f{i}_in"]).cuda()
        out, sf = ops.quantize(x, 0, 1, max_scale=2.25, precision="fp8e4m3",
                               swizzle=bool(int(z[f"f{i}_swizzle"])))
        np.testing.assert_array_equal(out.view(torch.uint8).cpu().numpy(), z[f"f{i}_out"])
        np.testing.assert_array_equal(sf.cpu().numpy(), z[f"f{i}_sf"])


def test_rowwise_zero_row_matches_reference_nan(ops):
    x = gaussian((4, 32), seed=2)
    x[2] = 0
    _check_rowwise(ops, x, "fp8e4m3")
    _check_rowwise(ops, x, "int8")


@pytest.mark.parametrize("precision", ["fp8e4m3", "int8"])
def test_full_size_config4_rowwise(ops, precision):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((32768, 8192), generator=g, device="cuda")
    mask = torch.rand((32768, 8192), generator=g, device="cuda") < 0.01
    x = torch.where(mask, x * 50.0, x).bfloat16()
    del mask
    out, sf = ops.quantize(x, 0, 1, precision=precision)
    for r0 in range(0, 32768, 4096):
        xs = x[r0:r0 + 4096]
        if precision == "fp8e4m3":
            ro, rsf = emu.quantize_fp8_ref(xs)
            assert torch.equal(out[r0:r0 + 4096].view(torch.uint8), ro.view(torch.uint8))
        else:
            ro, rsf = emu.quantize_int8_ref(xs)
            assert torch.equal(out[r0:r0 + 4096], ro)
        assert torch.equal(sf[r0:r0 + 4096], rsf)
