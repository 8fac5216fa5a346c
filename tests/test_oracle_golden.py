"""CPU tests: the restatement in oracle/ against the golden vectors produced by the
reference's own test oracles (tests/golden/make_golden.py), plus self-consistency."""
import os

import numpy as np
import pytest
import torch

from oracle import emulation as emu
from tests.helpers import bf16_from_bits, gaussian


def test_nvfp4_known_answer_vs_reference_get_ref(golden_dir):
    z = np.load(os.path.join(golden_dir, "nvfp4_quantize_known_answer.npz"))
    for i in range(int(z["n_cases"])):
        x = bf16_from_bits(z[f"q{i}_in"])
        cd, rd, sw = (int(v) for v in z[f"q{i}_meta"])
        packed, sf, g = emu.quantize_nvfp4_ref(x, cd, rd, swizzle=bool(sw))
        deq = emu.e2m1_codes_to_float(emu.unpack_fp4(packed))
        # the reference compares dequantised codes with atol 1e-3 (test_quantize_bench.py:189)
        np.testing.assert_allclose(deq.numpy(), z[f"q{i}_deq_codes"], atol=1e-3, rtol=1e-6)
        np.testing.assert_array_equal(sf.view(torch.uint8).numpy(), z[f"q{i}_sf"])
        np.testing.assert_allclose(g.numpy(), z[f"q{i}_g"], rtol=1e-6)


def test_linear_vs_reference_get_torch_results(golden_dir):
    z = np.load(os.path.join(golden_dir, "nvfp4_linear_reference_emulation.npz"))
    for i in range(int(z["n_cases"])):
        a = bf16_from_bits(z[f"l{i}_a"])
        b = bf16_from_bits(z[f"l{i}_b"])
        bias = None
        if f"l{i}_bias" in z:
            bias = torch.from_numpy(z[f"l{i}_bias"]).to(eval(str(z[f"l{i}_bias_dtype"])))
        odt = eval(str(z[f"l{i}_out_dtype"]))
        a4, asf, ag = emu.quantize_nvfp4_ref(a)
        b4, bsf, bg = emu.quantize_nvfp4_ref(b)
        out = emu.linear_nvfp4_ref(a4, asf, ag, b4, bsf, bg, bias=bias, out_dtype=odt)
        ref = torch.from_numpy(z[f"l{i}_out"])
        # the reference's own tolerance (test_linear_bench.py:152)
        torch.testing.assert_close(out.float(), ref, atol=1e-2, rtol=1e-2)
        # and the tighter bar of this build: relative L2
        rel = (out.float() - ref).norm() / ref.norm()
        assert rel < 2e-3, rel


def test_fp8_known_answer(golden_dir):
    z = np.load(os.path.join(golden_dir, "fp8_quantize_known_answer.npz"))
    for i in range(int(z["n_cases"])):
        x = bf16_from_bits(z[f"f{i}_in"])
        out, sf = emu.quantize_fp8_ref(x, 0, 1, 2.25, bool(int(z[f"f{i}_swizzle"])))
        np.testing.assert_array_equal(out.view(torch.uint8).numpy(), z[f"f{i}_out"])
        np.testing.assert_array_equal(sf.numpy(), z[f"f{i}_sf"])


def test_e4m3_encoder_matches_torch_cast():
    g = torch.Generator().manual_seed(1)
    x = torch.cat([torch.rand(200000, generator=g) * 500, torch.rand(100000, generator=g) * 0.05,
                   torch.tensor([0.0, 448.0, 449.0, 1e9, 2.0 ** -10, 2.0 ** -9, 3 * 2.0 ** -10])])
    mine = emu.e4m3_rne_sat_bits(x)
    ref = x.clamp(max=448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(mine, ref)
    allv = torch.arange(0, 127, dtype=torch.uint8)
    assert torch.equal(emu.e4m3_rne_sat_bits(emu.e4m3_bits_to_float(allv)), allv)
    assert int(emu.e4m3_rne_sat_bits(torch.tensor([float("nan")]))[0]) == 0x7F


def test_e2m1_thresholds_and_negative_zero():
    y = torch.tensor([0.0, -0.0, 0.25, 0.2500001, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.0001, 100.0,
                      -0.1, -0.75, -7.0])
    want = [0, 8, 0, 1, 2, 2, 4, 4, 6, 6, 7, 7, 8, 10, 15]
    assert emu.e2m1_rne_sat_codes(y).tolist() == want


def test_config1_properties():
    """BASELINE config 1: scale byte of the amax block saturates at 448, -0 codes exist,
    both scale layouts describe the same numbers."""
    A = gaussian((128, 512), seed=0)
    a, asf, ag = emu.quantize_nvfp4_ref(A)
    assert a.shape == (128, 256) and asf.shape == (8, 128, 4)
    assert int(asf.view(torch.uint8).max()) == 126
    assert int((emu.unpack_fp4(a) == 8).sum()) > 0
    a2, asf2, _ = emu.quantize_nvfp4_ref(A, sf_layout="128x4")
    assert asf2.shape == (1, 8, 32, 4, 4)
    assert torch.equal(a, a2)
    assert torch.equal(emu.dequantize_nvfp4_ref(a, asf, ag), emu.dequantize_nvfp4_ref(a2, asf2, ag))
    d = emu.dequantize_nvfp4_ref(a, asf, ag)
    rel = (d - A.float()).norm() / A.float().norm()
    assert rel < 0.2


def test_zero_tensor_and_zero_blocks():
    x = torch.zeros((16, 64), dtype=torch.bfloat16)
    p, sf, g = emu.quantize_nvfp4_ref(x)
    assert float(g) == 0 and int(p.max()) == 0 and int(sf.view(torch.uint8).max()) == 0
    x[3, 5] = 2.0
    x[4, 17] = -0.0
    p, sf, g = emu.quantize_nvfp4_ref(x)
    codes = emu.unpack_fp4(p)
    assert codes[3, 5] == 7 and codes[4, 17] == 8 and int((codes != 0).sum()) == 2


def test_int8_rounding():
    x = torch.tensor([[127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -127.0, 63.5] + [0.0] * 8]).bfloat16()
    q, sf = emu.quantize_int8_ref(x, 0, 1, 127)
    assert q[0, :8].tolist() == [127, 0, 2, 2, 0, -2, -127, 64]
    assert sf.shape == (16,) and float(sf[0]) == 1.0 and float(sf[1]) == 0.0


@pytest.mark.parametrize("shape,cd,rd", [((2, 3, 20, 70), 3, 1), ((5, 33, 17), 1, 2)])
def test_layout_roundtrip(shape, cd, rd):
    x = gaussian(shape, seed=3)
    p, sf, g = emu.quantize_nvfp4_ref(x, cd, rd)
    p2, sf2, _ = emu.quantize_nvfp4_ref(x, cd, rd, sf_layout="128x4")
    assert torch.equal(p, p2)
    m, k = shape[cd], shape[rd]
    lead = p.shape[:-2]
    pf, sff, sf2f = p.reshape(-1, *p.shape[-2:]), sf.reshape(-1, *sf.shape[-3:]), sf2.reshape(-1, *sf2.shape[-5:])
    for b in range(pf.shape[0]):
        r1 = emu.sf_ac4k_to_rows(sff[b].view(torch.uint8), m, emu.align_up(k, 64) // 16)
        r2 = emu.sf_tile128x4_to_rows(sf2f[b].view(torch.uint8), m, emu.align_up(k, 64) // 16)
        assert torch.equal(r1, r2)
    assert len(lead) == len(shape) - 2


def test_rope3d_vs_reference_oracle(golden_dir):
    """The restatement against outputs of the reference's own rope_params / rope_apply_reference
    (test/test_rope_3d_apply.py:5-42), bit for bit."""
    z = np.load(os.path.join(golden_dir, "rope3d_reference_oracle.npz"))
    for i in range(int(z["n_cases"])):
        x = bf16_from_bits(z[f"r{i}_x"])
        grid = torch.from_numpy(z[f"r{i}_grid"])
        freqs = torch.view_as_complex(torch.from_numpy(z[f"r{i}_freqs"]))
        assert torch.equal(torch.view_as_real(emu.rope_params_ref(int(z[f"r{i}_max_pos"]), x.shape[-1])),
                           torch.view_as_real(freqs))
        out = emu.rope3d_ref(x, grid, freqs)
        np.testing.assert_array_equal(out.view(torch.int16).numpy().view(np.uint16), z[f"r{i}_out"])
