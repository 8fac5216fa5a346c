"""INT8 x FP8 attention on B200: the block-of-tokens INT8 quantiser bit for bit against the restatement, the kernel
behind `mha_int8_x_fp8_fwd` against the tile-wise restatement on the same quantised operands, and
`attention(precision="int8+fp8e4m3")` against scaled_dot_product_attention at the bar and on the shapes of the
reference's test/test_attention_bench.py:18-63,67-176 (cosine similarity > 0.99, assert_close atol 2e-1 / rtol 1e-2)."""
import math

import pytest
import torch
import torch.nn.functional as F

from oracle import emulation as E

pytestmark = pytest.mark.gpu


def _ops():
    from ac4k_kernel_b200 import _cuda_ops
    from ac4k_kernel_b200.ops import attention, quantize
    from ac4k_kernel_b200.ops.attention import _int8_quantize
    return _cuda_ops, attention, quantize, _int8_quantize


def _cos(a, b):
    return F.cosine_similarity(a.float().flatten()[None], b.float().flatten()[None]).item()


def _sdp(q, k, v, layout):
    if layout == "BHND":
        return F.scaled_dot_product_attention(q, k, v)
    return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).contiguous()


def _qkv(B, Nq, Nkv, H, Dqk, Dv, layout, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    def mk(n, d):
        shape = (B, n, H, d) if layout == "BNHD" else (B, H, n, d)
        return torch.randn(shape, dtype=torch.bfloat16, device="cuda", generator=g)
    return mk(Nq, Dqk), mk(Nkv, Dqk), mk(Nkv, Dv)


@pytest.mark.parametrize("B,N,H,D,layout,block", [
    (1, 256, 1, 128, "BNHD", 64), (2, 100, 3, 128, "BNHD", 128), (2, 111, 2, 100, "BHND", 64), (3, 33, 2, 12, "BNHD", 64),
    (1, 70, 2, 65, "BHND", 16), (1, 200, 1, 256, "BNHD", 128), (1, 1, 1, 16, "BHND", 32),
])
def test_block_quantiser_bit_exact(B, N, H, D, layout, block):
    _, _, _, int8_quantize = _ops()
    g = torch.Generator(device="cuda").manual_seed(N * 7 + D)
    shape = (B, N, H, D) if layout == "BNHD" else (B, H, N, D)
    x = torch.randn(shape, dtype=torch.bfloat16, device="cuda", generator=g)
    if N > 40:
        (x[:, 32:40] if layout == "BNHD" else x[:, :, 32:40]).zero_()      # zero rows inside a block
    if N > 64 and block <= 64:
        (x[:, 64:64 + block] if layout == "BNHD" else x[:, :, 64:64 + block]).zero_()   # an all-zero block: scale 0, values 0
    y, s = int8_quantize(x, layout, 1 if layout == "BNHD" else 2, BLOCK_SIZE=block)
    ry, rs = E.quantize_int8_block_ref(x, layout, block)
    assert y.shape == ry.shape and s.shape == rs.shape
    assert torch.equal(s, rs)
    assert torch.equal(y, ry)


@pytest.mark.parametrize("layout,D", [("BNHD", 128), ("BHND", 100), ("BNHD", 12)])
def test_block_quantiser_with_subtraction(layout, D):
    """x - mean inside the quantiser = the quantiser on the bf16 tensor x - mean."""
    _, _, _, int8_quantize = _ops()
    g = torch.Generator(device="cuda").manual_seed(D)
    shape = (2, 300, 3, D) if layout == "BNHD" else (2, 3, 300, D)
    n_dim = 1 if layout == "BNHD" else 2
    x = torch.randn(shape, dtype=torch.bfloat16, device="cuda", generator=g) + 0.7
    mean = x.mean(dim=n_dim, keepdim=True)
    y0, s0 = int8_quantize(x - mean, layout, n_dim, BLOCK_SIZE=128)
    y1, s1 = int8_quantize(x, layout, n_dim, BLOCK_SIZE=128, sub=mean)
    assert torch.equal(y0, y1) and torch.equal(s0, s1)


# the shapes of the reference's test (the 75 600-token one with one head: 732 ms of fp32 SDPA, fine)
REF_CASES = [
    (1, 75600, 1, 128, "BNHD"), (1, 100, 1, 128, "BNHD"), (11, 100, 12, 12, "BNHD"), (11, 100, 12, 65, "BNHD"),
    (10, 330, 12, 100, "BNHD"), (1, 256, 1, 128, "BNHD"), (1, 128, 1, 128, "BNHD"), (2, 128, 3, 128, "BNHD"),
    (1, 33, 1, 128, "BNHD"), (1, 444, 1, 88, "BNHD"), (2, 111, 2, 100, "BHND"),
]


@pytest.mark.parametrize("B,N,H,D,layout", REF_CASES)
def test_attention_against_sdpa_at_the_reference_bar(B, N, H, D, layout):
    _, attention, _, _ = _ops()
    q, k, v = _qkv(B, N, N, H, D, D, layout, seed=9567 + N + D)
    o = attention(q, k, v, layout=layout, precision="int8+fp8e4m3")
    ref = _sdp(q, k, v, layout)
    assert o.shape == ref.shape and o.dtype == torch.bfloat16
    assert _cos(o, ref) > 0.99
    torch.testing.assert_close(o, ref, atol=2e-1, rtol=1e-2)


ORACLE_CASES = [
    # B, H, Nq, Nkv, Dqk, Dv
    (1, 1, 256, 256, 128, 128),
    (2, 3, 200, 200, 128, 128),
    (1, 2, 77, 515, 128, 128),       # Nq != Nkv, three keys in the last tile, ragged query tile
    (1, 2, 300, 129, 128, 128),      # one key in the second key tile; three query tiles
    (2, 2, 130, 190, 96, 80),        # head dimensions below 128
    (1, 3, 100, 100, 12, 12),
    (1, 1, 128, 2048, 128, 128),
]


@pytest.mark.parametrize("B,H,Nq,Nkv,Dqk,Dv", ORACLE_CASES)
@pytest.mark.parametrize("layout", ["BHND", "BNHD"])
def test_kernel_against_oracle_on_the_same_operands(B, H, Nq, Nkv, Dqk, Dv, layout):
    ops, _, quantize, int8_quantize = _ops()
    q, k, v = _qkv(B, Nq, Nkv, H, Dqk, Dv, layout, seed=31 * Nq + Nkv)
    n_dim = 1 if layout == "BNHD" else 2
    qq, qs = int8_quantize(q, layout, n_dim, BLOCK_SIZE=64)
    kq, ks = int8_quantize(k, layout, n_dim, BLOCK_SIZE=128)
    vq, vs = quantize(v, 3, n_dim, swizzle=True, max_scale=2.25, precision="fp8e4m3")
    sm = 1 / math.sqrt(Dqk)
    if layout == "BNHD":
        out = torch.full((B, Nq, H, Dv), float("nan"), dtype=torch.bfloat16, device="cuda")
        view = out.permute(0, 2, 1, 3)
    else:
        out = torch.full((B, H, Nq, Dv), float("nan"), dtype=torch.bfloat16, device="cuda")
        view = out
    ops.mha_int8_x_fp8_fwd(view, qq, qs, 64, kq, ks, 128, vq, vs, sm)
    torch.cuda.synchronize()
    from ac4k_kernel_b200 import _lib
    assert _lib.device_status() == 0
    want = E.mha_int8_x_fp8_ref(qq, qs, 64, kq, ks, 128, vq, vs, sm)
    got = view.float()
    assert torch.isfinite(got).all()
    # Tolerance, stated: exact integer scores on both sides; the kernel's ex2.approx / quartic against torch.exp2 move a few
    # roundings of P to e4m3, and the fp32 accumulation order differs: relative L2 error 2e-3, every element within
    # 2e-2 + 2 % of the value.
    rel = ((got - want.float()).norm() / want.float().norm()).item()
    assert rel < 2e-3, rel
    torch.testing.assert_close(got, want.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("q_block,k_block", [(16, 16), (32, 64), (128, 32), (64, 64)])
def test_other_quantisation_block_sizes(q_block, k_block):
    ops, _, quantize, int8_quantize = _ops()
    q, k, v = _qkv(2, 300, 333, 2, 128, 128, "BHND", seed=q_block + k_block)
    k = k * torch.linspace(0.2, 3.0, 333, device="cuda").bfloat16()[None, None, :, None]     # scales that differ along the keys
    qq, qs = int8_quantize(q, "BHND", 2, BLOCK_SIZE=q_block)
    kq, ks = int8_quantize(k, "BHND", 2, BLOCK_SIZE=k_block)
    vq, vs = quantize(v, 3, 2, swizzle=True, max_scale=2.25, precision="fp8e4m3")
    out = torch.empty((2, 2, 300, 128), dtype=torch.bfloat16, device="cuda")
    ops.mha_int8_x_fp8_fwd(out, qq, qs, q_block, kq, ks, k_block, vq, vs, 128 ** -0.5)
    want = E.mha_int8_x_fp8_ref(qq, qs, q_block, kq, ks, k_block, vq, vs, 128 ** -0.5)
    rel = ((out.float() - want.float()).norm() / want.float().norm()).item()
    assert rel < 2e-3, rel


def test_fp16_tile_accumulation_of_the_reference_is_within_the_same_bound():
    """The reference rounds each key tile's P V to fp16 before adding it to O; the restatement can do both."""
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn((1, 2, 300, 128), generator=g).bfloat16() for _ in range(3))
    qq, qs = E.quantize_int8_block_ref(q, "BHND", 64)
    kq, ks = E.quantize_int8_block_ref(k, "BHND", 128)
    vq, vs = E.quantize_fp8_ref(v, 3, 2, 2.25, swizzle=True)
    a = E.mha_int8_x_fp8_ref(qq, qs, 64, kq, ks, 128, vq, vs, 128 ** -0.5, out_dtype=torch.float32)
    b = E.mha_int8_x_fp8_ref(qq, qs, 64, kq, ks, 128, vq, vs, 128 ** -0.5, fp16_tile_accumulate=True, out_dtype=torch.float32)
    assert ((a - b).norm() / a.norm()).item() < 1e-3


def test_out_argument_repeatability_and_checks():
    ops, attention, quantize, int8_quantize = _ops()
    q, k, v = _qkv(2, 256, 256, 2, 128, 128, "BNHD", seed=5)
    out = torch.empty_like(q)
    r = attention(q, k, v, layout="BNHD", out=out)                 # the reference's default precision
    assert r.data_ptr() == out.data_ptr()
    assert torch.equal(out, attention(q, k, v, layout="BNHD", precision="int8+fp8e4m3"))
    qq, qs = int8_quantize(q, "BNHD", 1, BLOCK_SIZE=64)
    kq, ks = int8_quantize(k, "BNHD", 1, BLOCK_SIZE=128)
    vq, vs = quantize(v, 3, 1, swizzle=True, max_scale=2.25, precision="fp8e4m3")
    o = torch.empty((2, 2, 256, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):      # scale count does not match the block size
        ops.mha_int8_x_fp8_fwd(o, qq, qs, 128, kq, ks, 128, vq, vs, 0.1)
    with pytest.raises(RuntimeError):      # a block size that is not a power of two
        ops.mha_int8_x_fp8_fwd(o, qq, qs, 64, kq, ks[..., :1].expand(2, 2, 6).contiguous(), 48, vq, vs, 0.1)
    with pytest.raises(RuntimeError):
        ops.mha_int8_x_fp8_fwd(o.float(), qq, qs, 64, kq, ks, 128, vq, vs, 0.1)
    with pytest.raises(RuntimeError):
        ops.mha_int8_x_fp8_fwd(o, qq, qs, 64, kq, ks, 128, vq.view(torch.uint8), vs, 0.1)
