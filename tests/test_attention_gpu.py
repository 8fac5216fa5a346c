"""NVFP4 attention on B200: the kernel behind `mha_nvfp4_fwd` against the tile-wise restatement in
oracle/emulation.py on the same quantised operands, and `attention(precision="nvfp4")` against
scaled_dot_product_attention at the bar of the reference's test/test_attention_bench.py:18-63,177-190
(cosine similarity > 0.98, assert_close atol 2e-1 / rtol 1e-1)."""
import math

import pytest
import torch
import torch.nn.functional as F

from oracle import emulation as E

pytestmark = pytest.mark.gpu


def _ops():
    from ac4k_kernel_b200 import _cuda_ops
    from ac4k_kernel_b200.ops import attention, quantize
    return _cuda_ops, attention, quantize


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


# the two nvfp4 cases of the reference's test at the reference's bar
@pytest.mark.parametrize("B,N,H,D,layout", [(1, 256, 1, 128, "BNHD"), (1, 64, 1, 128, "BNHD")])
def test_attention_against_sdpa_at_the_reference_bar(B, N, H, D, layout):
    _, attention, _ = _ops()
    q, k, v = _qkv(B, N, N, H, D, D, layout, seed=9567 + N)
    o = attention(q, k, v, layout=layout, precision="nvfp4")
    ref = _sdp(q, k, v, layout)
    assert o.shape == ref.shape and o.dtype == torch.bfloat16
    assert _cos(o, ref) > 0.98
    torch.testing.assert_close(o, ref, atol=2e-1, rtol=1e-1)


# Ragged, multi-head, both layouts, long.  Same cosine bar; the element-wise bound is the reference's with the
# absolute part widened to 0.35: over a few hundred thousand outputs of short sequences the 4-bit error of single
# elements reaches 0.25 in the CPU restatement as well (the reference tests one head of 64 and 256 keys only).
SDP_CASES = [
    (1, 128, 1, 128, "BHND"),
    (2, 200, 3, 128, "BNHD"),
    (2, 333, 4, 128, "BHND"),
    (1, 1, 2, 128, "BNHD"),
    (1, 1000, 2, 100, "BNHD"),
    (1, 4096, 2, 128, "BHND"),
    (2, 512, 4, 64, "BNHD"),
]


@pytest.mark.parametrize("B,N,H,D,layout", SDP_CASES)
def test_attention_against_sdpa_more_shapes(B, N, H, D, layout):
    _, attention, _ = _ops()
    q, k, v = _qkv(B, N, N, H, D, D, layout, seed=9567 + N)
    o = attention(q, k, v, layout=layout, precision="nvfp4")
    ref = _sdp(q, k, v, layout)
    assert o.shape == ref.shape and o.dtype == torch.bfloat16
    assert _cos(o, ref) > 0.98
    torch.testing.assert_close(o, ref, atol=3.5e-1, rtol=1e-1)


ORACLE_CASES = [
    # B, H, Nq, Nkv, Dqk, Dv
    (1, 1, 256, 256, 128, 128),
    (1, 1, 64, 64, 128, 128),
    (2, 3, 200, 200, 128, 128),
    (1, 2, 77, 515, 128, 128),       # Nq != Nkv, ragged last key tile (3 keys), ragged query tile
    (1, 2, 300, 129, 128, 128),      # one key in the second key tile; three query tiles (the last CTA has one)
    (1, 1, 40, 64, 128, 128),        # a single key tile, half of it
    (1, 2, 130, 190, 96, 80),        # head dimensions below 128 (padded by the quantiser)
    (1, 1, 128, 2048, 128, 128),
    (2, 2, 150, 300, 64, 64),        # one K = 64 step over the head dimension
    (1, 3, 100, 100, 48, 16),
    (1, 2, 260, 140, 128, 32),
]


@pytest.mark.parametrize("B,H,Nq,Nkv,Dqk,Dv", ORACLE_CASES)
@pytest.mark.parametrize("layout", ["BHND", "BNHD"])
@pytest.mark.parametrize("sf_layout", ["128x4", "ac4k"])
def test_kernel_against_oracle_on_the_same_operands(B, H, Nq, Nkv, Dqk, Dv, layout, sf_layout):
    ops, _, quantize = _ops()
    q, k, v = _qkv(B, Nq, Nkv, H, Dqk, Dv, layout, seed=17 * Nq + Nkv)
    n_dim = 1 if layout == "BNHD" else 2
    qq, qs, qg = quantize(q, n_dim, 3, sf_layout=sf_layout)
    kq, ks, kg = quantize(k, n_dim, 3, sf_layout=sf_layout)
    vq, vs, vg = quantize(v, 3, n_dim, swizzle=True, sf_layout=sf_layout)
    sm = 1 / math.sqrt(Dqk)
    if layout == "BNHD":
        out = torch.full((B, Nq, H, Dv), float("nan"), dtype=torch.bfloat16, device="cuda")
        view = out.permute(0, 2, 1, 3)
    else:
        out = torch.full((B, H, Nq, Dv), float("nan"), dtype=torch.bfloat16, device="cuda")
        view = out
    ops.mha_nvfp4_fwd(view, qq, qs, qg, kq, ks, kg, vq, vs, vg, sm)
    torch.cuda.synchronize()
    from ac4k_kernel_b200 import _lib
    assert _lib.device_status() == 0
    # the restatement walks the keys in tiles of 128, as the kernel and the reference's kernel do (the tile decides which
    # running maximum P is rounded against: tests/test_attention_oracle.py)
    want = E.mha_nvfp4_ref(qq, qs, qg, kq, ks, kg, vq, vs, vg, sm, Nkv, tile=128)
    got = view.float()
    assert torch.isfinite(got).all()
    # Tolerance, stated: the kernel and the restatement differ in fp32 accumulation order, in ex2.approx
    # against torch.exp2 (2 ulp) and therefore in a few roundings of P to e2m1; relative L2 error 2e-3 and every
    # element within 2e-2 + 2 % of the value.
    rel = ((got - want.float()).norm() / want.float().norm()).item()
    assert rel < 2e-3, rel
    torch.testing.assert_close(got, want.float(), atol=2e-2, rtol=2e-2)


def test_both_scale_layouts_give_the_same_bytes():
    """The reference's call, verbatim (python/ac4k_kernel/ops/attention.py:113-128: default scale layout), against the
    tiled layout that `attention()` here asks the quantiser for."""
    ops, _, quantize = _ops()
    q, k, v = _qkv(2, 333, 200, 3, 128, 128, "BNHD", seed=11)
    outs = []
    for sf_layout in ("ac4k", "128x4"):
        qq, qs, qg = quantize(q, 1, 3, sf_layout=sf_layout)
        kq, ks, kg = quantize(k, 1, 3, sf_layout=sf_layout)
        vq, vs, vg = quantize(v, 3, 1, swizzle=True, sf_layout=sf_layout)
        o = torch.empty((2, 333, 3, 128), dtype=torch.bfloat16, device="cuda")
        ops.mha_nvfp4_fwd(o.permute(0, 2, 1, 3), qq, qs, qg, kq, ks, kg, vq, vs, vg, 128 ** -0.5)
        outs.append(o)
    assert torch.equal(outs[0], outs[1])


def test_out_argument_and_repeatability():
    _, attention, _ = _ops()
    q, k, v = _qkv(2, 256, 256, 2, 128, 128, "BNHD", seed=5)
    out = torch.empty_like(q)
    r = attention(q, k, v, layout="BNHD", precision="nvfp4", out=out)
    assert r.data_ptr() == out.data_ptr()
    again = attention(q, k, v, layout="BNHD", precision="nvfp4")
    assert torch.equal(out, again)


def test_argument_checks():
    ops, attention, quantize = _ops()
    q, k, v = _qkv(1, 64, 64, 1, 128, 128, "BHND", seed=1)
    qq, qs, qg = quantize(q, 2, 3, sf_layout="128x4")
    kq, ks, kg = quantize(k, 2, 3, sf_layout="128x4")
    vq, vs, vg = quantize(v, 3, 2, swizzle=True, sf_layout="128x4")
    o = torch.empty((1, 1, 64, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):      # output dtype
        ops.mha_nvfp4_fwd(o.float(), qq, qs, qg, kq, ks, kg, vq, vs, vg, 0.1)
    with pytest.raises(RuntimeError):      # K with another head dimension
        ops.mha_nvfp4_fwd(o, qq, qs, qg, kq[..., :32].contiguous(), ks, kg, vq, vs, vg, 0.1)
    with pytest.raises(RuntimeError):      # V over another number of keys
        ops.mha_nvfp4_fwd(o, qq, qs, qg, kq, ks, kg, torch.cat([vq, vq], dim=-1), vs, vg, 0.1)
    with pytest.raises(RuntimeError):      # scale layouts must agree
        q5 = quantize(q, 2, 3)[1]
        ops.mha_nvfp4_fwd(o, qq, q5, qg, kq, ks, kg, vq, vs, vg, 0.1)
    with pytest.raises(RuntimeError):      # head dimension above 128
        q256, k256, v256 = _qkv(1, 64, 64, 1, 256, 256, "BHND", seed=2)
        attention(q256, k256, v256, layout="BHND", precision="nvfp4")
    with pytest.raises(AssertionError):
        attention(q, k, v, layout="BHND", precision="fp16")
