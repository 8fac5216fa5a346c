"""CPU tests (gloo, world size 2) of the column-parallel plumbing: shard bounds, the all-reduce
of the global scale, the all-gather and its [M, N] view.  The local GEMM is stood in for by the
oracle so the test needs no GPU; on the GPU the same functions wrap the CUDA `linear`."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import emulation as emu
from tests.helpers import gaussian


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ac4k_kernel_b200 import parallel
        m, n, k = 48, 256, 128
        x = gaussian((m, k), seed=1)
        w = gaussian((n, k), seed=2, std=0.02)
        w[200, 5] = 3.0                      # the tensor amax lives in the LAST shard
        lo, hi = parallel.shard_bounds(n, rank, world)
        w_shard = w[lo:hi]
        # global scale of the whole weight from per-shard scales
        g = emu.global_scale_ref(w_shard).clone()
        parallel.allreduce_max_scale(g)
        assert torch.equal(g, emu.global_scale_ref(w)), (float(g), float(emu.global_scale_ref(w)))
        x4, xsf, xg = emu.quantize_nvfp4_ref(x)
        w4, wsf, _ = emu.quantize_nvfp4_ref(w_shard, global_scale=g)
        local = emu.linear_nvfp4_ref(x4, xsf, xg, w4, wsf, g)
        gathered = parallel.gather_columns(local)
        full = parallel.columns_view(gathered)
        # single-process result on the whole weight
        W4, Wsf, Wg = emu.quantize_nvfp4_ref(w)
        ref = emu.linear_nvfp4_ref(x4, xsf, xg, W4, Wsf, Wg)
        assert gathered.shape == (world, m, n // world)
        assert torch.equal(full, ref)
        # the shard's packed bytes are exactly the matching rows of the full quantisation
        assert torch.equal(w4, W4[lo:hi])
        results[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        results[rank] = repr(e)
    finally:
        dist.destroy_process_group()


def test_column_parallel_world2():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


def test_shard_bounds():
    from ac4k_kernel_b200 import parallel
    assert parallel.shard_bounds(28672, 3, 8) == (3 * 3584, 4 * 3584)
    assert parallel.shard_bounds(28672, 1, 2) == (14336, 28672)
    with pytest.raises(ValueError):
        parallel.shard_bounds(1000, 0, 8)


def test_single_process_gather_is_identity():
    from ac4k_kernel_b200 import parallel
    x = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    g = parallel.gather_columns(x)
    assert torch.equal(parallel.columns_view(g), x)
