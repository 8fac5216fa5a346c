"""A bounded device-side wait that runs out: the kernel must leave through its normal exit, report a status
code, and the context must stay usable.

The reference spins without a limit (lib/cuda/sm120/linear_nvfp4.cu:280-292: a stage that never arrives hangs
the GPU).  Here every wait carries a limit (2 s by default) that is an argument of the launch.  This test uses
the debug-hook build of the library (`build.py --hooks`, -DAC4K_DEBUG_HOOKS; the shipped library has neither the
switch nor the symbols): it shortens the limit to 3 ms and makes the CTA-pair kernel's producer leave out the
loads of its first stage, so that nothing ever arrives on that stage's barrier.  No trap, no bad address, no
endless loop: the MMA issuer's wait expires, then the producer's and the epilogue's, each role falls through to
the common exit, tensor memory is released, and `ac4k_device_status` returns AC4K_ERR_TIMEOUT with the code.
A normal GEMM on the same context right after gives the same bytes as the shipped library.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOOKS = os.path.join(ROOT, "ac4k_kernel_b200", "build_hooks", "libac4k_b200_hooks.so")


@pytest.mark.skipif(not os.path.exists(HOOKS), reason="debug-hook build not present (python ac4k_kernel_b200/build.py --hooks)")
def test_expired_wait_reports_status_and_context_survives():
    from ac4k_kernel_b200 import _lib, ops
    hooks = ctypes.CDLL(HOOKS)
    for name, (res, args) in _lib.SIGNATURES.items():
        fn = getattr(hooks, name)
        fn.restype, fn.argtypes = res, args
    hooks.ac4k_debug_set_wait_ns.argtypes = [ctypes.c_uint64]
    hooks.ac4k_debug_set_flags.argtypes = [ctypes.c_int]

    m = n = k = 512
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn((m, k), generator=g, device="cuda").bfloat16()
    b = (torch.randn((n, k), generator=g, device="cuda") * 0.02).bfloat16()
    a4, asf, ag = ops.quantize(a, 0, 1, sf_layout="128x4")
    b4, bsf, bg = ops.quantize(b, 0, 1, sf_layout="128x4")
    want = ops.linear(a4, asf, ag, b4, bsf, bg)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream

    def gemm(lib, out):
        return lib.ac4k_linear_nvfp4(out.data_ptr(), 0, a4.data_ptr(), asf.data_ptr(), ag.data_ptr(), b4.data_ptr(),
                                     bsf.data_ptr(), bg.data_ptr(), None, 0, m, n, k, 1, stream)

    status = ctypes.c_uint32(0)
    assert hooks.ac4k_device_status(ctypes.byref(status), 1) == 0 and status.value == 0
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    try:
        hooks.ac4k_debug_set_wait_ns(3_000_000)          # 3 ms per wait
        hooks.ac4k_debug_set_flags(256)                  # the first stage of cluster 0 is never loaded
        assert gemm(hooks, out) == 0                     # the launch itself succeeds: it is asynchronous
        rc = hooks.ac4k_device_status(ctypes.byref(status), 1)
    finally:
        hooks.ac4k_debug_set_flags(0)
        hooks.ac4k_debug_set_wait_ns(0)
    assert rc == -7, rc                                  # AC4K_ERR_TIMEOUT
    assert status.value in (0xA1, 0xA2, 0xA3, 0xA4), hex(status.value)
    assert b"bounded device-side wait expired" in hooks.ac4k_last_error()
    # the word was cleared, the context answers, and the same library computes the GEMM correctly again
    assert hooks.ac4k_device_status(ctypes.byref(status), 1) == 0 and status.value == 0
    out2 = torch.zeros_like(out)
    assert gemm(hooks, out2) == 0
    torch.cuda.synchronize()
    assert hooks.ac4k_device_status(ctypes.byref(status), 1) == 0 and status.value == 0
    assert torch.equal(out2, want)
    # ... and so does the shipped library, which shares the context
    assert torch.equal(ops.linear(a4, asf, ag, b4, bsf, bg), want)
    assert _lib.device_status() == 0
