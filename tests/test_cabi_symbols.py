"""CPU test: the built library exports every symbol that include/ac4k_b200.h declares, and
the Python mirror exposes the reference module's names.  No compute call is made."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ac4k_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ac4k_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    from ac4k_kernel_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    syms = declared_symbols()
    assert "ac4k_linear_nvfp4" in syms and "ac4k_quantize_nvfp4" in syms
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in the header but not exported"
    assert set(_lib.SIGNATURES) == set(syms)


def test_no_measurement_switches_in_the_default_build():
    """The experiment switches (`ac4k_debug_set_*`) exist only in builds with -DAC4K_DEBUG_HOOKS; the library
    that ships must not export them."""
    import subprocess
    from ac4k_kernel_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in ("ac4k_debug_set_flags", "ac4k_debug_set_splits", "ac4k_debug_set_tile_n", "ac4k_debug_set_trace"):
        assert not hasattr(lib, name), f"{name} is exported by the default build"
    exported = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    assert "ac4k_debug" not in exported


def test_module_mirrors_reference_names():
    import ac4k_kernel_b200 as pkg
    from ac4k_kernel_b200 import _cuda_ops
    for name in ("mha_nvfp4_fwd", "mha_int8_x_fp8_fwd", "quantize_nvfp4", "quantize_fp8",
                 "quantize_int8", "linear_nvfp4", "rope3d", "__arch__", "__backend__",
                 "__arch_description__", "__version__"):
        assert hasattr(_cuda_ops, name)
    assert pkg.get_arch() == "sm100" and pkg.get_backend() == "cuda"
    assert not hasattr(_cuda_ops, "_out_of_scope")       # every name of the reference module is implemented


def test_argument_errors_without_gpu():
    """Rejected arguments return negative codes before anything touches the device."""
    from ac4k_kernel_b200._lib import LIB, last_error
    shape = (ctypes.c_int64 * 4)(1, 1, 16, 64)
    stride = (ctypes.c_int64 * 4)(0, 0, 64, 1)
    assert LIB.ac4k_quantize_nvfp4(None, None, None, None, shape, stride, 0, 0, None) == -1
    assert "NULL" in last_error()
    assert LIB.ac4k_quantize_nvfp4(8, 8, 16, 16, shape, stride, 0, 7, None) == -4
    assert LIB.ac4k_global_scale_bf16(None, -1, 1.0, 8, None) == -2
    assert LIB.ac4k_rope3d(8, 8, 8, 16, 1, 4, 2, 7, 4, None) == -2          # odd feature dimension
    assert LIB.ac4k_rope3d(None, 8, 8, 16, 1, 4, 2, 8, 4, None) == -1
    assert LIB.ac4k_rope3d(8, 8, 8, 16, 1, 4, 2, 4096, 4, None) == -5       # feature dimension above what is built
    sh = (ctypes.c_int64 * 4)(1, 1, 8, 16)
    assert LIB.ac4k_quantize_int8_block(8, 8, 8, sh, sh, 48, None, None, None) == -2         # block not a power of two
    assert LIB.ac4k_quantize_int8_block(None, 8, 8, sh, sh, 64, None, None, None) == -1
    o4 = (ctypes.c_int64 * 4)(1, 1, 1, 1)
    assert LIB.ac4k_mha_int8_x_fp8_fwd(16, o4, 16, 16, 64, 16, 16, 48, 16, 16, 1, 1, 8, 8, 128, 128, 0.1, None) == -5   # K block 48
    assert LIB.ac4k_mha_int8_x_fp8_fwd(16, o4, 16, 16, 64, 16, 16, 128, 16, 16, 1, 1, 8, 8, 256, 128, 0.1, None) == -5  # head dim 256
    assert LIB.ac4k_mha_nvfp4_fwd(16, o4, 16, 16, 16, 16, 16, 16, 16, 16, 16, 1, 1, 8, 8, 192, 128, 0.1, 1, None) == -5
    assert LIB.ac4k_mha_nvfp4_fwd(16, o4, 16, 16, 16, 16, 16, 16, 16, 16, 16, 1, 1, 8, 0, 128, 128, 0.1, 1, None) == -2
    assert LIB.ac4k_mha_nvfp4_fwd(16, o4, 16, 16, 16, 16, 16, 16, 16, 16, 16, 1, 1, 8, 8, 128, 128, -1.0, 1, None) == -5
    bad = (ctypes.c_int64 * 4)(1, 1, -3, 64)
    assert LIB.ac4k_quantize_fp8(8, 8, 16, 16, bad, stride, 0, None) == -2


def test_python_checks_mirror_reference():
    import torch
    from ac4k_kernel_b200 import _cuda_ops
    x = torch.zeros((16, 64), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _cuda_ops.quantize_nvfp4(torch.zeros((16, 32), dtype=torch.uint8),
                                 torch.zeros((1, 16, 4), dtype=torch.float8_e4m3fn), x,
                                 torch.zeros(()), 0, 1, False)


def test_gemm_argument_errors_without_gpu():
    """The GEMM entry points (plain, allocation-free, gather, re-quantising) reject bad sizes,
    codes, alignments and NULLs with negative codes and a message, before any CUDA call."""
    from ac4k_kernel_b200._lib import LIB, last_error
    P = 4096                                   # any 16-byte-aligned non-NULL value; never dereferenced
    lin = lambda fn, *a: fn(*a)
    # (D, d_dtype, A, A_sf, A_gs, B, B_sf, B_gs, bias, bias_dtype, M, N, K, sf_layout, stream)
    for fn in (LIB.ac4k_linear_nvfp4, LIB.ac4k_linear_nvfp4_noalloc):
        assert fn(P, 0, P, P, P, P, P, P, None, 0, -1, 8, 64, 0, None) == -2          # negative M
        assert fn(P, 9, P, P, P, P, P, P, None, 0, 8, 8, 64, 0, None) == -4           # unknown d_dtype
        assert fn(P, 0, P, P, P, P, P, P, None, 0, 8, 8, 64, 5, None) == -4           # unknown sf_layout
        assert fn(P, 0, P, P, P, P, P, P, None, 0, 0, 8, 64, 0, None) == 0            # empty output: nothing to do
        assert fn(None, 0, P, P, P, P, P, P, None, 0, 8, 8, 64, 0, None) == -1        # NULL D
        assert fn(P, 0, P, P, P, P, P, P, None, 0, 8, 8, 80, 0, None) == -2           # K not a multiple of 64
        assert "multiple of 64" in last_error()
        assert fn(P + 4, 0, P, P, P, P, P, P, None, 0, 8, 8, 64, 0, None) == -3       # misaligned D
    dst = (ctypes.c_void_p * 2)(P, P)
    g = LIB.ac4k_linear_nvfp4_gather
    # (D_dsts, n_dst, ldd, col_off, d_dtype, A, A_sf, A_gs, B, B_sf, B_gs, bias, bias_dtype, M, N, K, layout, stream)
    assert g(None, 1, 64, 0, 0, P, P, P, P, P, P, None, 0, 8, 64, 64, 1, None) == -1
    assert g(dst, 0, 64, 0, 0, P, P, P, P, P, P, None, 0, 8, 64, 64, 1, None) == -2        # no destination
    assert g(dst, 9, 64, 0, 0, P, P, P, P, P, P, None, 0, 8, 64, 64, 1, None) == -2        # more than 8
    assert g(dst, 2, 64, 8, 0, P, P, P, P, P, P, None, 0, 8, 64, 64, 1, None) == -2        # columns do not fit
    assert g(dst, 2, 132, 4, 0, P, P, P, P, P, P, None, 0, 8, 64, 64, 1, None) == -3       # ldd / col_off not % 8
    bad = (ctypes.c_void_p * 2)(P, None)
    assert g(bad, 2, 64, 0, 0, P, P, P, P, P, P, None, 0, 8, 64, 64, 1, None) == -1        # NULL destination
    r = LIB.ac4k_linear_nvfp4_requant
    # (out_fp4, out_sf, out_gs, out_layout, A, A_sf, A_gs, B, B_sf, B_gs, bias, bias_dtype, M, N, K, layout, stream)
    assert r(None, P, P, 1, P, P, P, P, P, P, None, 0, 8, 64, 64, 1, None) == -1
    assert r(P, P, P, 3, P, P, P, P, P, P, None, 0, 8, 64, 64, 1, None) == -4              # unknown output layout
    assert r(P, P, P, 1, P, P, P, P, P, P, None, 0, 8, 96, 64, 1, None) == -5              # N not a multiple of 64
    assert "64" in last_error()
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    assert LIB.ac4k_peer_alloc(0, ctypes.byref(ptr), handle) == -2
    assert LIB.ac4k_peer_alloc(1024, None, handle) == -1
    assert LIB.ac4k_peer_open(None, ctypes.byref(ptr)) == -1
    assert LIB.ac4k_peer_close(None) == 0 and LIB.ac4k_peer_free(None) == 0


def test_header_is_valid_c_and_links_from_c(tmp_path):
    """include/ac4k_b200.h compiled by a C compiler (not C++), linked against the built library and
    run: identity strings and argument rejections through the C ABI, no Python in between."""
    import shutil
    import subprocess
    from ac4k_kernel_b200 import _lib
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    exe = str(tmp_path / "use_from_c")
    src = os.path.join(ROOT, "tests", "c_abi", "use_from_c.c")
    libdir = os.path.dirname(_lib.LIB_PATH)
    cmd = [gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), src, "-o", exe,
           "-L", libdir, "-l:libac4k_b200.so", f"-Wl,-rpath,{libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stdout + r.stderr
