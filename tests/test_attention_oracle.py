"""The CPU restatement of NVFP4 attention (oracle/emulation.py) against fp32 scaled_dot_product_attention at the
bar of the reference's test/test_attention_bench.py:18-63,177-190.  The reference's kernel is sm_120a CUDA and
cannot run here, so this bar (the reference's own acceptance test) is what pins the restatement."""
import pytest
import torch
import torch.nn.functional as F

from oracle import emulation as E


def _sdp(q, k, v, layout):
    if layout == "BHND":
        return F.scaled_dot_product_attention(q.float(), k.float(), v.float())
    return F.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                                          v.transpose(1, 2).float()).transpose(1, 2)


@pytest.mark.parametrize("B,N,H,D,layout", [(1, 256, 1, 128, "BNHD"), (1, 64, 1, 128, "BNHD"), (2, 150, 2, 100, "BHND")])
def test_restatement_meets_the_reference_bar(B, N, H, D, layout):
    g = torch.Generator().manual_seed(9567)
    shape = (B, N, H, D) if layout == "BNHD" else (B, H, N, D)
    q, k, v = (torch.randn(shape, generator=g).bfloat16() for _ in range(3))
    o = E.attention_nvfp4_ref(q, k, v, layout)
    ref = _sdp(q, k, v, layout)
    assert o.shape == ref.shape
    cos = F.cosine_similarity(o.float().flatten()[None], ref.flatten()[None]).item()
    assert cos > 0.98
    torch.testing.assert_close(o.float(), ref, atol=2e-1 if H == 1 else 3.5e-1, rtol=1e-1)


def test_tile_size_only_changes_rounding():
    """Walking the keys in tiles of 64 or 128 changes the running maximum P is taken against and with it the 4-bit
    rounding of P (a few percent per element), nothing else: the two results agree to the size of that noise."""
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn((1, 1, 200, 128), generator=g).bfloat16() for _ in range(3))
    qq, qs, qg = E.quantize_nvfp4_ref(q, 2, 3, sf_layout="128x4")
    kq, ks, kg = E.quantize_nvfp4_ref(k, 2, 3, sf_layout="128x4")
    vq, vs, vg = E.quantize_nvfp4_ref(v, 3, 2, swizzle=True, sf_layout="128x4")
    a = E.mha_nvfp4_ref(qq, qs, qg, kq, ks, kg, vq, vs, vg, 128 ** -0.5, 200, tile=128, out_dtype=torch.float32)
    b = E.mha_nvfp4_ref(qq, qs, qg, kq, ks, kg, vq, vs, vg, 128 ** -0.5, 200, tile=64, out_dtype=torch.float32)
    assert ((a - b).norm() / a.norm()).item() < 5e-2


@pytest.mark.parametrize("B,N,H,D,layout", [(1, 256, 1, 128, "BNHD"), (1, 100, 1, 128, "BNHD"), (3, 100, 2, 12, "BNHD"),
                                             (2, 111, 2, 100, "BHND")])
def test_int8_x_fp8_restatement_meets_the_reference_bar(B, N, H, D, layout):
    """test/test_attention_bench.py:67-176: cosine > 0.99, assert_close atol 2e-1 / rtol 1e-2 against SDPA."""
    g = torch.Generator().manual_seed(9567)
    shape = (B, N, H, D) if layout == "BNHD" else (B, H, N, D)
    q, k, v = (torch.randn(shape, generator=g).bfloat16() for _ in range(3))
    o = E.attention_int8_x_fp8_ref(q, k, v, layout)
    ref = _sdp(q, k, v, layout)
    cos = F.cosine_similarity(o.float().flatten()[None], ref.flatten()[None]).item()
    assert cos > 0.99
    torch.testing.assert_close(o.float(), ref, atol=2e-1, rtol=1e-2)


def test_int8_block_quantiser_restatement():
    x = torch.tensor([[1.0, -2.0, 0.5, 127.0], [3.0, 0.0, -127.0, 63.4]]).bfloat16().reshape(1, 1, 2, 4)
    y, s = E.quantize_int8_block_ref(x, "BHND", 16)
    assert y.shape == (1, 1, 2, 16) and s.shape == (1, 1, 1) and s.item() == 1.0
    assert y[0, 0, :, :4].tolist() == [[1, -2, 0, 127], [3, 0, -127, 63]]      # truncation toward zero
    assert (y[..., 4:] == 0).all()
    z, sz = E.quantize_int8_block_ref(torch.zeros((1, 20, 2, 8), dtype=torch.bfloat16), "BNHD", 16)
    assert (z == 0).all() and (sz == 0).all() and sz.shape == (1, 2, 2)
