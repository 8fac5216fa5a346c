"""Generate the golden vectors under tests/golden/ from the reference's OWN test oracles.

Run once where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/ac4k_kernel

The reference's tests need an sm_120 GPU and its compiled `_cuda_ops`; neither exists on a
B200 box.  Their *oracle* halves, however, are plain torch:

  * `test/test_quantize_bench.py::get_ref`       (NVFP4 quantiser, known-answer inputs)
  * `test/test_quantize_bench.py::qunatize_fp8`  (per-token FP8, exact equality)
  * `test/test_linear_bench.py::get_torch_results` (dequantise -> fp32 matmul -> cast)
  * `test/test_rope_3d_apply.py::rope_params`, `::rope_apply_reference` (3-D rotary embedding;
    `python tests/golden/make_golden.py <checkout> rope` writes only that fixture)

This script imports those files with `ac4k_kernel.ops` replaced by a stub, redirects their
hard-coded "cuda" allocations to the CPU, runs them on seeded inputs and stores inputs and
outputs as .npz.  It also runs the reference's own assertions with the stub bound to the
restatement in oracle/emulation.py, i.e. the reference's test code is what validates the
restatement.  Nothing here is needed at test time; the tests only read the .npz files.
"""
import importlib.util
import os
import random
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import emulation as emu  # noqa: E402


def _cpu_factories():
    """Make torch factory calls ignore device="cuda" and Tensor.cuda() a no-op."""
    for name in ("empty", "randn", "tensor", "zeros", "full", "randint"):
        orig = getattr(torch, name)

        def wrapped(*a, __orig=orig, **kw):
            if kw.get("device") in ("cuda", torch.device("cuda")):
                kw.pop("device")
            return __orig(*a, **kw)

        setattr(torch, name, wrapped)
    torch.Tensor.cuda = lambda self, *a, **k: self


def _stub_ops():
    """`from ac4k_kernel.ops import quantize, linear` resolves to the restatement."""

    def quantize(input, cross_dim, reduce_dim, max_scale=None, precision="nvfp4",
                 swizzle=False, output=None, sf=None):
        if precision == "nvfp4":
            return emu.quantize_nvfp4_ref(input, cross_dim, reduce_dim, swizzle=swizzle)
        if precision == "fp8e4m3":
            return emu.quantize_fp8_ref(input, cross_dim, reduce_dim,
                                        448.0 if max_scale is None else max_scale, swizzle)
        return emu.quantize_int8_ref(input, cross_dim, reduce_dim,
                                     127 if max_scale is None else max_scale)

    def linear(x, xs, xg, w, ws, wg, bias=None, out=None):
        dt = torch.bfloat16 if out is None else out.dtype
        return emu.linear_nvfp4_ref(x, xs, xg, w, ws, wg, bias=bias, out_dtype=dt)

    pkg = types.ModuleType("ac4k_kernel")
    ops = types.ModuleType("ac4k_kernel.ops")
    ops.quantize, ops.linear = quantize, linear
    ops.rope3d = lambda x, grid_sizes, freqs, output=None: emu.rope3d_ref(x, grid_sizes, freqs)
    pkg.ops = ops
    sys.modules["ac4k_kernel"] = pkg
    sys.modules["ac4k_kernel.ops"] = ops


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits16(t):
    return t.view(torch.int16).numpy().view(np.uint16)


def rope_golden(ref_root):
    """Outputs of the reference's rope_params / rope_apply_reference on seeded inputs."""
    tr = _load(os.path.join(ref_root, "test", "test_rope_3d_apply.py"), "ref_test_rope")
    g = torch.Generator().manual_seed(9567)
    cases = [(2, 70, 3, 16, [(3, 4, 5), (2, 5, 7)], 16),       # one batch entry padded, one full
             (1, 24, 2, 20, [(2, 3, 4)], 8),                   # C = 10: 4 + 3 + 3 pairs, D not a multiple of 8
             (1, 40, 2, 128, [(2, 4, 5)], 32),
             (2, 36, 1, 6, [(1, 1, 1), (3, 3, 4)], 4)]         # C = 3: one pair per axis; a grid of a single position
    out = {}
    for i, (b, s, n, d, grids, max_pos) in enumerate(cases):
        x = torch.randn((b, s, n, d), generator=g).bfloat16()
        gs = torch.tensor(grids, dtype=torch.int32)
        fr = tr.rope_params(max_pos, d)
        y = tr.rope_apply_reference(x, gs, fr)
        assert torch.equal(y.view(torch.int16), emu.rope3d_ref(x, gs, fr).view(torch.int16))
        out[f"r{i}_x"] = bits16(x)
        out[f"r{i}_grid"] = gs.numpy()
        out[f"r{i}_max_pos"] = np.array(max_pos)
        out[f"r{i}_freqs"] = torch.view_as_real(fr).numpy()
        out[f"r{i}_out"] = bits16(y)
    out["n_cases"] = np.array(len(cases))
    np.savez_compressed(os.path.join(HERE, "rope3d_reference_oracle.npz"), **out)
    print("rope3d golden vectors written")


def main(ref_root, only=None):
    _cpu_factories()
    _stub_ops()
    if only == "rope":
        rope_golden(ref_root)
        return
    tq = _load(os.path.join(ref_root, "test", "test_quantize_bench.py"), "ref_test_quantize")
    tl = _load(os.path.join(ref_root, "test", "test_linear_bench.py"), "ref_test_linear")

    # 1. the reference's assertions, with the restatement standing in for the kernels
    torch.manual_seed(9567)
    random.seed(9527)
    tq.qunatize_fp8((64, 48), 0, 1)
    tq.qunatize_fp8((2, 70, 5, 32), 3, 1, swizzle=True)
    tq.qunatize_fp8((100, 10), 0, 1)
    tq.qunatize_fp8((16, 16), 0, 1, swizzle=True)
    tq.qunatize_fp8((77, 79), 0, 1, swizzle=True)
    tq.test_quantize_bench((96, 80), 1, 0)
    tq.test_quantize_bench((128, 512), 0, 1)
    tq.test_random_bennch(6)
    for shape in [(128, 128, 128), (10, 512, 512), (130, 384, 256), (123, 321, 256),
                  (10, 15, 512), (1, 4, 256), (64, 64, 128), (12, 23, 55)]:
        tl.test_linear(torch.bfloat16, shape)
    tl.test_linear(torch.bfloat16, (12, 23, 5), o_dtype=torch.float32)
    tl.test_linear(torch.bfloat16, (2, 3, 51), o_dtype=torch.float16, bias_type=torch.float32)
    tl.test_linear(torch.bfloat16, (5, 3, 51), o_dtype=torch.bfloat16, bias_type=torch.float32)
    print("reference assertions passed against the restatement")

    # 2. golden vectors: outputs of the reference's get_ref on known-answer inputs
    vals = torch.tensor([1.0, 2.0, 4.0, 6.0, -1.0, -2.0, -4.0, -6.0], dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(9567)
    cases = [((128, 512), 0, 1, False), ((96, 80), 1, 0, False), ((37, 200), 0, 1, True),
             ((50, 33), 1, 0, True), ((3, 20, 70), 1, 2, False), ((2, 3, 40, 24), 3, 1, True)]
    out = {}
    for i, (shape, cd, rd, sw) in enumerate(cases):
        x = vals[torch.randint(0, len(vals), shape, generator=g)]
        o, sf, gs = tq.get_ref(x, cd, rd, sw)
        out[f"q{i}_in"] = bits16(x)
        out[f"q{i}_meta"] = np.array([cd, rd, int(sw)], dtype=np.int64)
        out[f"q{i}_deq_codes"] = o.numpy().astype(np.float32)
        out[f"q{i}_sf"] = sf.view(torch.uint8).numpy()
        out[f"q{i}_g"] = gs.numpy().astype(np.float32)
    out["n_cases"] = np.array(len(cases))
    np.savez_compressed(os.path.join(HERE, "nvfp4_quantize_known_answer.npz"), **out)

    # 3. golden vectors: the reference's dequantise+matmul on quantised operands.
    #    Operands come from the restatement (validated in step 1); the stored result is the
    #    reference's own get_torch_results.
    out = {}
    g = torch.Generator().manual_seed(0)
    lin_cases = [(128, 256, 512, None, None), (10, 15, 512, None, None),
                 (123, 321, 256, None, None), (12, 23, 55, None, None),
                 (5, 3, 51, torch.float32, torch.bfloat16), (2, 33, 51, torch.float32, torch.float32)]
    for i, (m, n, k, bt, ot) in enumerate(lin_cases):
        a = torch.randn((m, k), generator=g).bfloat16()
        b = torch.randn((n, k), generator=g).bfloat16()
        bias = None if bt is None else torch.randn((1, n), generator=g).to(bt)
        a4, asf, ag = emu.quantize_nvfp4_ref(a)
        b4, bsf, bg = emu.quantize_nvfp4_ref(b)
        ref = tl.get_torch_results(a4, b4, asf, bsf, 1 / ag, 1 / bg, m, n, 16, o_dtype=ot,
                                   bias=bias)
        out[f"l{i}_a"] = bits16(a)
        out[f"l{i}_b"] = bits16(b)
        if bias is not None:
            out[f"l{i}_bias"] = bias.float().numpy()
            out[f"l{i}_bias_dtype"] = np.array(str(bt))
        out[f"l{i}_out"] = ref.float().numpy()
        out[f"l{i}_out_dtype"] = np.array(str(ref.dtype))
    out["n_cases"] = np.array(len(lin_cases))
    np.savez_compressed(os.path.join(HERE, "nvfp4_linear_reference_emulation.npz"), **out)

    # 4. FP8 per-token known answers: the reference test's own expected tensors
    #    (re-derived with its formulas on its value set, max_scale 2.25).
    out = {}
    g = torch.Generator().manual_seed(9567)
    v8 = torch.tensor([-8, -6, -5, -4, 1, 2, 3, 4, 5, 6, 8, 9], dtype=torch.bfloat16)
    for i, (shape, sw) in enumerate([((64, 48), False), ((77, 79), True), ((100, 10), False)]):
        x = v8[torch.randint(0, len(v8), shape, generator=g)]
        m, k = shape
        kp, m16 = emu.align_up(k, 16), emu.align_up(m, 16)
        xp = torch.nn.functional.pad(x, (0, kp - k, 0, m16 - m))
        if sw:
            xp = xp.reshape(-1, 2, 4, 2).permute(0, 2, 1, 3).contiguous().reshape(m16, kp)
        amax = xp.abs().amax(dim=-1, keepdim=True).float()
        sf_ref = amax.squeeze(-1) / 2.25
        o_ref = (xp.float() / amax * 2.25).to(torch.float8_e4m3fn)[:m]
        out[f"f{i}_in"] = bits16(x)
        out[f"f{i}_swizzle"] = np.array(int(sw))
        out[f"f{i}_out"] = o_ref.view(torch.uint8).numpy()
        out[f"f{i}_sf"] = sf_ref.numpy()
    out["n_cases"] = np.array(3)
    np.savez_compressed(os.path.join(HERE, "fp8_quantize_known_answer.npz"), **out)
    rope_golden(ref_root)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of ac4k_kernel> [rope]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else None)
