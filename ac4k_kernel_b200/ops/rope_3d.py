"""`rope3d()`: 3-D rotary position embedding on B200.

Same signature and module layout as the reference's python/ac4k_kernel/ops/rope_3d.py:18-58.
"""
from typing import Optional

import torch

from .. import _cuda_ops

rope3d_kernel = _cuda_ops.rope3d


class Ac4kRoPEOp(torch.nn.Module):

    def forward(self, x, grid_sizes, freqs, output=None):
        if output is None:
            output = torch.empty_like(x)
        rope3d_kernel(x, grid_sizes, freqs, output)
        return output


_OP = Ac4kRoPEOp()


def rope3d(x: torch.Tensor, grid_sizes: torch.Tensor, freqs: torch.Tensor,
           output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x: [B, S, N, D] bf16; grid_sizes: [B, 3] int32 (frames, height, width); freqs: [max_pos, D // 2] complex128;
    output: optional [B, S, N, D] bf16.  Returns output (positions behind a batch entry's grid are copied from x)."""
    return _OP(x, grid_sizes, freqs, output=output)
