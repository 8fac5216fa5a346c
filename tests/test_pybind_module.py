"""The compiled pybind11 `_cuda_ops` module (csrc/bindings_pybind.cc, built by `build.py --pybind`): the
reference's module name, function names, positional signatures (include/ac4k_kernel/ops.h:13-54) and module
attributes (lib/cuda_bindings.cc:37-44), over the same C ABI as the ctypes mirror.  CPU: it imports and rejects
bad arguments like the reference's TORCH_CHECKs; GPU: it gives the same bytes as the ctypes path."""
import pytest
import torch


@pytest.fixture(scope="module")
def mod():
    from ac4k_kernel_b200.native import load
    return load()


def test_names_and_attributes(mod):
    for name in ("mha_nvfp4_fwd", "mha_int8_x_fp8_fwd", "quantize_nvfp4", "quantize_fp8", "quantize_int8",
                 "linear_nvfp4", "rope3d"):
        assert callable(getattr(mod, name))
    assert mod.__name__.endswith("_cuda_ops")
    assert mod.__arch__ == "sm100" and mod.__backend__ == "cuda" and mod.__version__ == "0.1.0"
    assert "Blackwell" in mod.__arch_description__


def test_checks_raise_like_torch_check(mod):
    x = torch.zeros((16, 64), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        mod.quantize_nvfp4(torch.zeros((16, 32), dtype=torch.uint8), torch.zeros((1, 16, 4), dtype=torch.float8_e4m3fn),
                           x, torch.zeros(()), 0, 1, False)
    with pytest.raises(RuntimeError, match="2d matrix"):
        mod.linear_nvfp4(torch.zeros(4), x, x, x, x, x, x, None)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        mod.rope3d(x, x, x, x)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        mod.mha_int8_x_fp8_fwd(x, x, x, 64, x, x, 128, x, x, 0.1)


@pytest.mark.gpu
def test_same_bytes_as_the_ctypes_path(mod):
    from ac4k_kernel_b200 import _cuda_ops as ct
    g = torch.Generator(device="cuda").manual_seed(3)
    m, n, k = 300, 520, 1024
    a = torch.randn((m, k), generator=g, device="cuda").bfloat16()
    b = (torch.randn((n, k), generator=g, device="cuda") * 0.02).bfloat16()
    gs = {}
    for name, t in (("a", a), ("b", b)):
        out = torch.empty((), dtype=torch.float32, device="cuda")
        mod.global_scale_bf16(out, t, 2688.0)
        gs[name] = out
    quant = {}
    for which, fn in (("pybind", mod), ("ctypes", ct)):
        for layout in ("ac4k", "128x4"):
            for name, t in (("a", a), ("b", b)):
                rows = t.shape[0]
                p4 = torch.empty((rows, k // 2), dtype=torch.uint8, device="cuda")
                shape = (k // 64, (rows + 15) // 16 * 16, 4) if layout == "ac4k" else ((rows + 127) // 128, k // 64, 32, 4, 4)
                sf = torch.zeros(shape, dtype=torch.float8_e4m3fn, device="cuda")
                fn.quantize_nvfp4(p4, sf, t, gs[name], 0, 1, False)
                quant[which, layout, name] = (p4, sf)
    for layout in ("ac4k", "128x4"):
        for name in ("a", "b"):
            assert torch.equal(quant["pybind", layout, name][0], quant["ctypes", layout, name][0])
            assert torch.equal(quant["pybind", layout, name][1].view(torch.uint8), quant["ctypes", layout, name][1].view(torch.uint8))
        a4, asf = quant["pybind", layout, "a"]
        b4, bsf = quant["pybind", layout, "b"]
        for odt in (torch.bfloat16, torch.float16, torch.float32):
            bias = torch.randn((1, n), generator=g, device="cuda").to(odt)
            d1 = torch.empty((m, n), dtype=odt, device="cuda")
            d2 = torch.empty_like(d1)
            mod.linear_nvfp4(d1, a4, asf, gs["a"], b4, bsf, gs["b"], bias)
            ct.linear_nvfp4(d2, a4, asf, gs["a"], b4, bsf, gs["b"], bias)
            assert torch.equal(d1, d2)
        d1 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        d2 = torch.empty_like(d1)
        mod.linear_nvfp4(d1, a4, asf, gs["a"], b4, bsf, gs["b"], None)
        ct.linear_nvfp4(d2, a4, asf, gs["a"], b4, bsf, gs["b"], None)
        assert torch.equal(d1, d2)
    # per-row FP8 / INT8
    for name, odt, smax in (("quantize_fp8", torch.float8_e4m3fn, torch.tensor(448.0, device="cuda")),
                            ("quantize_int8", torch.int8, torch.tensor(127, dtype=torch.int32, device="cuda"))):
        res = []
        for fn in (mod, ct):
            out = torch.empty((m, k), dtype=odt, device="cuda")
            sf = torch.zeros(((m + 15) // 16 * 16,), dtype=torch.float32, device="cuda")
            if name == "quantize_fp8":
                getattr(fn, name)(out, sf, a, smax, 0, 1, False)
            else:
                getattr(fn, name)(out, sf, a, smax, 0, 1)
            res.append((out, sf))
        assert torch.equal(res[0][0].view(torch.uint8), res[1][0].view(torch.uint8)) and torch.equal(res[0][1], res[1][1])
    torch.cuda.synchronize()


@pytest.mark.gpu
def test_attention_same_bytes_as_the_ctypes_path(mod):
    from ac4k_kernel_b200 import _cuda_ops as ct
    from ac4k_kernel_b200.ops import quantize
    g = torch.Generator(device="cuda").manual_seed(4)
    B, N, H, D = 2, 200, 3, 128
    q, k, v = (torch.randn((B, N, H, D), generator=g, device="cuda").bfloat16() for _ in range(3))
    qq, qs, qg = quantize(q, 1, 3, sf_layout="128x4")
    kq, ks, kg = quantize(k, 1, 3, sf_layout="128x4")
    vq, vs, vg = quantize(v, 3, 1, swizzle=True, sf_layout="128x4")
    outs = []
    for fn in (mod, ct):
        o = torch.empty((B, N, H, D), dtype=torch.bfloat16, device="cuda")
        fn.mha_nvfp4_fwd(o.permute(0, 2, 1, 3), qq, qs, qg, kq, ks, kg, vq, vs, vg, D ** -0.5)
        outs.append(o)
    assert torch.equal(outs[0], outs[1])
    with pytest.raises(RuntimeError, match="5D tensor"):      # scale layouts must agree: q_sf decides
        mod.mha_nvfp4_fwd(outs[0].permute(0, 2, 1, 3), qq, quantize(q, 1, 3)[1], qg, kq, ks, kg, vq, vs, vg, 0.1)
