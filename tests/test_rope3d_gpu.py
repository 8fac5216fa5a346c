"""3-D rotary position embedding on B200 against the golden vectors of the reference's own Python oracle and against
the restatement in oracle/emulation.py; bit-exact (fp64 products, one rounding to fp32, one to bf16)."""
import os

import numpy as np
import pytest
import torch

from oracle import emulation as emu
from tests.helpers import bf16_from_bits

pytestmark = pytest.mark.gpu


def _rope():
    from ac4k_kernel_b200.ops import rope3d
    return rope3d


def test_golden_vectors_of_the_reference_oracle(golden_dir):
    rope3d = _rope()
    z = np.load(os.path.join(golden_dir, "rope3d_reference_oracle.npz"))
    for i in range(int(z["n_cases"])):
        x = bf16_from_bits(z[f"r{i}_x"]).cuda()
        grid = torch.from_numpy(z[f"r{i}_grid"]).cuda()
        freqs = torch.view_as_complex(torch.from_numpy(z[f"r{i}_freqs"])).cuda()
        out = rope3d(x, grid, freqs)
        np.testing.assert_array_equal(out.cpu().view(torch.int16).numpy().view(np.uint16), z[f"r{i}_out"])


@pytest.mark.parametrize("B,grids,S,N,D,max_pos", [
    (1, [(4, 6, 10)], 240, 5, 128, 64),
    (3, [(2, 3, 4), (1, 1, 1), (3, 5, 7)], 105, 2, 64, 16),      # ragged: 24, 1 and 105 of 105 positions
    (2, [(2, 2, 2), (0, 3, 3)], 16, 3, 20, 8),                   # D % 8 != 0 (pairwise path); an empty grid
    (1, [(3, 4, 5)], 60, 1, 2, 8),                               # a single complex pair per head
    (1, [(2, 3, 4)], 24, 7, 256, 8),
    (2, [(2, 3, 4), (2, 2, 5)], 24, 3, 24, 8),                   # C = 12 does not divide 1024: factors staged in shared memory
    (1, [(9, 2, 2)], 36, 2, 16, 4),                              # frame index past the table: its last row is used
])
def test_against_the_restatement(B, grids, S, N, D, max_pos):
    rope3d = _rope()
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + D)
    x = torch.randn((B, S, N, D), dtype=torch.bfloat16, device="cuda", generator=g)
    grid = torch.tensor(grids, dtype=torch.int32, device="cuda")
    freqs = emu.rope_params_ref(max_pos, D).cuda()
    out = torch.full_like(x, float("nan"))
    res = rope3d(x, grid, freqs, out)
    assert res.data_ptr() == out.data_ptr()
    # an index past the table reads its last row (the reference would read out of bounds): restate that by padding
    # the table with copies of its last row
    need = max(max(g_) for g_ in grids)
    table = freqs if need <= max_pos else torch.cat([freqs, freqs[-1:].expand(need - max_pos, -1)])
    want = emu.rope3d_ref(x, grid, table)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))


def test_the_shape_of_the_reference_test():
    """[1, 21 * 45 * 80 = 75600, 40, 128] with a 1024-row table (test/test_rope_3d_apply.py:49-56), against the restatement
    evaluated on the GPU, and the reference's own tolerance (atol 1e-2) as a second, weaker statement."""
    rope3d = _rope()
    F_, H_, W_ = 21, 45, 80
    x = torch.randn((1, F_ * H_ * W_, 40, 128), dtype=torch.bfloat16, device="cuda",
                    generator=torch.Generator(device="cuda").manual_seed(9567))
    grid = torch.tensor([[F_, H_, W_]], dtype=torch.int32, device="cuda")
    freqs = emu.rope_params_ref(1024, 128).cuda()
    out = rope3d(x, grid, freqs)
    want = emu.rope3d_ref(x, grid, freqs)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    torch.testing.assert_close(out.float(), want.float(), rtol=0.0, atol=1e-2)
    # rotation: every complex pair keeps its modulus up to the two roundings
    a = torch.view_as_complex(x[:, :4096].float().reshape(1, 4096, 40, 64, 2)).abs()
    b = torch.view_as_complex(out[:, :4096].float().reshape(1, 4096, 40, 64, 2)).abs()
    assert ((a - b).abs() <= 0.01 * a + 1e-3).all()


def test_special_values():
    """Zeros of both signs, bf16 subnormals, the largest finite values and infinities go through the widening to fp64
    exactly; NaNs stay NaNs."""
    rope3d = _rope()
    bits = torch.tensor([0x0000, 0x8000, 0x0001, 0x807f, 0x0040, 0x0080, 0x7f7f, 0xff7f, 0x7f80, 0xff80, 0x3f80, 0xc2f7],
                        dtype=torch.int32).to(torch.int16)
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, bits.numel(), (1, 24, 2, 128), generator=g)
    x = bits[idx].view(torch.bfloat16).cuda()
    grid = torch.tensor([[2, 3, 4]], dtype=torch.int32, device="cuda")
    freqs = emu.rope_params_ref(8, 128).cuda()
    out = rope3d(x, grid, freqs)
    want = emu.rope3d_ref(x, grid, freqs)
    nan = torch.isnan(want.float())
    assert torch.equal(torch.isnan(out.float()), nan)
    assert torch.equal(out.view(torch.int16)[~nan], want.view(torch.int16)[~nan])
    x[0, 0, 0, 0] = float("nan")
    assert torch.isnan(rope3d(x, grid, freqs)[0, 0, 0, :2].float()).all()


def test_argument_checks():
    from ac4k_kernel_b200 import _cuda_ops
    x = torch.randn((1, 8, 2, 16), dtype=torch.bfloat16, device="cuda")
    grid = torch.tensor([[2, 2, 2]], dtype=torch.int32, device="cuda")
    freqs = emu.rope_params_ref(4, 16).cuda()
    out = torch.empty_like(x)
    with pytest.raises(RuntimeError):
        _cuda_ops.rope3d(x.float(), grid, freqs, out)
    with pytest.raises(RuntimeError):
        _cuda_ops.rope3d(x, grid.long(), freqs, out)
    with pytest.raises(RuntimeError):
        _cuda_ops.rope3d(x, grid, freqs.to(torch.complex64), out)
    with pytest.raises(RuntimeError):
        _cuda_ops.rope3d(x, grid[:, :2].contiguous(), freqs, out)
    with pytest.raises(RuntimeError):
        _cuda_ops.rope3d(x, grid, freqs, out[:, :4].contiguous())
    with pytest.raises(RuntimeError):
        _cuda_ops.rope3d(x, grid, freqs[:, :4].contiguous(), out)
