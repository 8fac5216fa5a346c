"""Times the reference's own quantiser and RoPE kernels (built for sm_100a by oracle/build_ref.py) beside this
repository's on the same device tensors and prints one line per kernel; the figures in
profiles/reference_kernels_on_b200.md come from it.  Test-side tooling: not imported by the package.

    python tests/reference_kernels_compare.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import build_ref, emulation as E          # noqa: E402
from ac4k_kernel_b200 import _cuda_ops, ops            # noqa: E402
from ac4k_kernel_b200.ops.quant import _global_scale   # noqa: E402


def timed(fn, n=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(n):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / n * 1e-3


def main():
    ref = build_ref.load()
    if ref is None:
        print("oracle/_ref is not built")
        return 1
    m, k = 32768, 8192                                   # the quantiser configuration of the benchmark: 512 MiB of bf16
    x = torch.randn((m, k), dtype=torch.bfloat16, device="cuda")
    gs = _global_scale(x, 6.0 * 448.0)
    out, sf, _ = ops.quantize(x, 0, 1)
    r_out, r_sf = torch.empty_like(out), torch.empty_like(sf)
    nbytes = x.numel() * 2 + out.numel() + sf.numel()
    t_ref = timed(lambda: ref.quantize_nvfp4(r_out, r_sf, x, gs, 0, 1, False))
    t_own = timed(lambda: _cuda_ops.quantize_nvfp4(out, sf, x, gs, 0, 1, False))
    diff = int((out != r_out).sum()) + int((sf.view(torch.uint8) != r_sf.view(torch.uint8)).sum())
    print(f"quantize_nvfp4 [{m}, {k}]: reference kernel {t_ref * 1e6:.1f} us = {nbytes / t_ref / 1e9:.0f} GB/s; "
          f"this repository {t_own * 1e6:.1f} us = {nbytes / t_own / 1e9:.0f} GB/s; speed-up {t_ref / t_own:.2f}; "
          f"bytes differing: {diff} of {out.numel() + sf.numel()}")
    for prec in ("fp8e4m3", "int8"):
        o, s = ops.quantize(x, 0, 1, precision=prec)
        ro, rs = torch.empty_like(o), torch.empty_like(s)
        if prec == "fp8e4m3":
            smax = torch.tensor(448.0, device="cuda")
            t_ref = timed(lambda: ref.quantize_fp8(ro, rs, x, smax, 0, 1, False))
        else:
            smax = torch.tensor(127, dtype=torch.int32, device="cuda")
            t_ref = timed(lambda: ref.quantize_int8(ro, rs, x, smax, 0, 1))
        t_own = timed(lambda: ops.quantize(x, 0, 1, precision=prec, output=o, sf=s))
        nb = x.numel() * 3 + s.numel() * 4
        diff = int((o.view(torch.uint8) != ro.view(torch.uint8)).sum())
        print(f"quantize_{prec} [{m}, {k}]: reference kernel {t_ref * 1e6:.1f} us = {nb / t_ref / 1e9:.0f} GB/s; "
              f"this repository {t_own * 1e6:.1f} us = {nb / t_own / 1e9:.0f} GB/s; speed-up {t_ref / t_own:.2f}; "
              f"bytes differing (fast-math division in the reference): {diff} of {o.numel()}")
    del x, out, sf, r_out, r_sf, o, s, ro, rs
    # the quantisers as attention calls them (python/ac4k_kernel/ops/attention.py:102-135, 157-186): [B, N, H, D] tensors,
    # q / k along the head dimension, V along the tokens with the K permutation
    v = torch.randn((1, 75600, 40, 128), dtype=torch.bfloat16, device="cuda")
    for name, cd, rd, sw in (("q / k: cross N, reduce D", 1, 3, False), ("V: cross D, reduce N, swizzle", 3, 1, True)):
        out, sf, gs = ops.quantize(v, cd, rd, swizzle=sw)
        r_out, r_sf = torch.empty_like(out), torch.empty_like(sf)
        t_ref = timed(lambda: ref.quantize_nvfp4(r_out, r_sf, v, gs, cd, rd, sw), n=5)
        t_own = timed(lambda: _cuda_ops.quantize_nvfp4(out, sf, v, gs, cd, rd, sw))
        diff = int((out != r_out).sum()) + int((sf.view(torch.uint8) != r_sf.view(torch.uint8)).sum())
        print(f"quantize_nvfp4 [1, 75600, 40, 128] {name}: reference kernel {t_ref * 1e6:.1f} us; this repository "
              f"{t_own * 1e6:.1f} us; speed-up {t_ref / t_own:.2f}; bytes differing: {diff} of {out.numel() + sf.numel()}")
    o, s = ops.quantize(v, 3, 1, swizzle=True, max_scale=2.25, precision="fp8e4m3")
    ro, rs = torch.empty_like(o), torch.empty_like(s)
    smax = torch.tensor(2.25, device="cuda")
    t_ref = timed(lambda: ref.quantize_fp8(ro, rs, v, smax, 3, 1, True), n=5)
    t_own = timed(lambda: ops.quantize(v, 3, 1, swizzle=True, max_scale=2.25, precision="fp8e4m3", output=o, sf=s))
    diff = int((o.view(torch.uint8) != ro.view(torch.uint8)).sum())
    print(f"quantize_fp8 [1, 75600, 40, 128] V: cross D, reduce N, swizzle, scale_max 2.25: reference kernel {t_ref * 1e6:.1f} us; "
          f"this repository {t_own * 1e6:.1f} us; speed-up {t_ref / t_own:.2f}; bytes differing: {diff} of {o.numel()}")
    del v, out, sf, r_out, r_sf, o, s, ro, rs
    b, f, h, w, n, d = 1, 21, 45, 80, 40, 128
    xr = torch.randn((b, f * h * w, n, d), dtype=torch.bfloat16, device="cuda")
    grid = torch.tensor([[f, h, w]], dtype=torch.int32, device="cuda")
    freqs = E.rope_params_ref(1024, d).cuda()
    y_ref, y_own = torch.empty_like(xr), torch.empty_like(xr)
    t_ref = timed(lambda: ref.rope3d(xr, grid, freqs, y_ref), n=5)
    t_own = timed(lambda: ops.rope3d(xr, grid, freqs, output=y_own))
    nb = xr.numel() * 4
    print(f"rope3d [{b}, {f * h * w}, {n}, {d}]: reference kernel {t_ref * 1e6:.1f} us = {nb / t_ref / 1e9:.0f} GB/s; "
          f"this repository {t_own * 1e6:.1f} us = {nb / t_own / 1e9:.0f} GB/s; speed-up {t_ref / t_own:.2f}; "
          f"bytes equal: {torch.equal(y_ref, y_own)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
