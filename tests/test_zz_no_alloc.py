"""GPU test of `ac4k_linear_nvfp4_noalloc`, the entry point for hosts that may not allocate device
memory while running (a plugin inside another process's fixed memory budget, a serving loop that
bans allocator calls).  It is called through the C ABI exactly like `ac4k_linear_nvfp4` and must
give the same bytes; its split-K scratch is a fixed 8 MiB array inside the library instead of a
stream-ordered allocation.  Two calls in a row share that array, so the second call also checks
that nothing left behind by the first one leaks into the result.

Collected last on purpose (file name): a failure here cannot hide the other tests in a run that
stops at the first failure.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _call(fn, out, a4, asf, ag, b4, bsf, bg, bias, layout):
    m, n = out.shape
    k = a4.shape[1] * 2
    rc = fn(out.data_ptr(), DT[out.dtype], a4.data_ptr(), asf.data_ptr(), ag.data_ptr(), b4.data_ptr(),
            bsf.data_ptr(), bg.data_ptr(), None if bias is None else bias.data_ptr(),
            0 if bias is None else DT[bias.dtype], m, n, k, layout, torch.cuda.current_stream().cuda_stream)
    return rc


def _operands(m, n, k, seed, layout):
    from ac4k_kernel_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((m, k), generator=g, device="cuda").bfloat16()
    b = (torch.randn((n, k), generator=g, device="cuda") * 0.02).bfloat16()
    return ops.quantize(a, 0, 1, sf_layout=layout) + ops.quantize(b, 0, 1, sf_layout=layout)


@pytest.mark.parametrize("layout_name,layout", [("128x4", 1), ("ac4k", 0)])
def test_noalloc_matches_regular_entry_point_twice(layout_name, layout):
    from ac4k_kernel_b200._lib import LIB, device_status, last_error
    # decode-shaped and split-K problems back to back
    # (the first runs unsplit, the second adds its two K slices inside the kernel - neither needs scratch;
    # the last one is cut into 8 slices whose partial sums, 8 x 200 x 1024 fp32 = 6.25 MiB, use the array)
    cases = [(16, 2048, 4096, torch.bfloat16, None), (64, 8192, 8192, torch.float16, torch.float32),
             (256, 1024, 4096, torch.float32, None), (200, 1024, 8192, torch.float32, torch.bfloat16)]
    for i, (m, n, k, odt, bdt) in enumerate(cases):
        a4, asf, ag, b4, bsf, bg = _operands(m, n, k, 40 + i, layout_name)
        bias = None if bdt is None else torch.randn((1, n), device="cuda").to(bdt)
        ref = torch.full((m, n), float("nan"), dtype=odt, device="cuda")
        out = torch.full((m, n), float("nan"), dtype=odt, device="cuda")
        assert _call(LIB.ac4k_linear_nvfp4, ref, a4, asf, ag, b4, bsf, bg, bias, layout) == 0, last_error()
        assert _call(LIB.ac4k_linear_nvfp4_noalloc, out, a4, asf, ag, b4, bsf, bg, bias, layout) == 0, last_error()
        torch.cuda.synchronize()
        assert device_status() == 0
        assert not bool(torch.isnan(out.float()).any())
        # same kernels, same order of additions: the results are identical, which is well inside the
        # tolerance of the GEMM tests (relative L2 2e-3, 2 ulps)
        assert torch.equal(out, ref), float((out.float() - ref.float()).abs().max())


def test_noalloc_large_shape_needs_no_scratch():
    """Shapes that do not split K run unchanged (nothing to take from the fixed array)."""
    from ac4k_kernel_b200._lib import LIB, last_error
    a4, asf, ag, b4, bsf, bg = _operands(512, 1024, 1024, 7, "128x4")
    ref = torch.empty((512, 1024), dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(ref)
    assert _call(LIB.ac4k_linear_nvfp4, ref, a4, asf, ag, b4, bsf, bg, None, 1) == 0, last_error()
    assert _call(LIB.ac4k_linear_nvfp4_noalloc, out, a4, asf, ag, b4, bsf, bg, None, 1) == 0, last_error()
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


def test_noalloc_rejects_scratch_beyond_its_maximum():
    """[8 slices, 128, 2304] fp32 = 9 MiB of partial sums does not fit the 8 MiB array."""
    from ac4k_kernel_b200._lib import LIB, last_error
    a4, asf, ag, b4, bsf, bg = _operands(128, 2304, 8192, 9, "128x4")
    out = torch.empty((128, 2304), dtype=torch.bfloat16, device="cuda")
    rc = _call(LIB.ac4k_linear_nvfp4_noalloc, out, a4, asf, ag, b4, bsf, bg, None, 1)
    assert rc == -2 and "exceeds the fixed scratch" in last_error()
    # the regular entry point handles the same shape
    assert _call(LIB.ac4k_linear_nvfp4, out, a4, asf, ag, b4, bsf, bg, None, 1) == 0, last_error()
    torch.cuda.synchronize()
