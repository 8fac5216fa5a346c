"""Column-parallel NVFP4 linear on two GPUs (one process per GPU, NCCL): the fused all-gather
epilogue and the pipelined send/recv exchange must both reproduce the NCCL all-gather result,
which in turn equals the single-GPU GEMM over the whole weight.  Skipped with fewer than two GPUs.
"""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, result_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    try:
        from ac4k_kernel_b200 import ops, parallel
        from tests.helpers import gaussian
        x = gaussian((m, k), seed=11).cuda()
        w = (gaussian((n, k), seed=12) * 0.02).bfloat16().cuda()       # every rank builds the whole weight ...
        lo, hi = parallel.shard_bounds(n, rank, world)
        x4, xsf, xg = ops.quantize(x, 0, 1, sf_layout="128x4")
        w4, wsf, wg = parallel.quantize_weight_shard(w[lo:hi].contiguous(), None, "128x4")   # ... but quantises its shard
        # single-GPU result over the whole weight (the global scale of the whole tensor is what the shards used)
        f4, fsf, fg = ops.quantize(w, 0, 1, sf_layout="128x4")
        assert torch.equal(fg, wg)
        whole = ops.linear(x4, xsf, xg, f4, fsf, fg)
        # (1) NCCL all-gather
        gathered, local = parallel.column_parallel_linear(x4, xsf, xg, w4, wsf, wg)
        assert torch.equal(parallel.columns_view(gathered), whole)
        # (2) pipelined send/recv
        g2 = torch.zeros_like(gathered)
        parallel.column_parallel_linear_pipelined(x4, xsf, xg, w4, wsf, wg, g2, chunks=2)
        torch.cuda.synchronize()
        assert torch.equal(g2, gathered)
        # (3) fused epilogue stores into every rank's [M, N] buffer.  The activations change every step and a
        # consumer kernel reads this rank's copy between the steps (one rank is slowed down on purpose), so a
        # step that overwrote a buffer another rank still reads would show up as a wrong checksum.
        peer = parallel.PeerOutput(m, n, torch.bfloat16)
        for t in peer.tensors:
            t.fill_(-3.0)
        torch.cuda.synchronize()
        dist.barrier()
        steps = 6
        xs = [gaussian((m, k), seed=100 + i).cuda() for i in range(steps)]
        xq = [ops.quantize(v, 0, 1, sf_layout="128x4") for v in xs]
        wholes = [ops.linear(q[0], q[1], q[2], f4, fsf, fg) for q in xq]
        sums, fulls_ok = [], []
        spin = torch.empty((4096, 4096), device="cuda")
        for i in range(steps):
            full = parallel.column_parallel_linear_fused(xq[i][0], xq[i][1], xq[i][2], w4, wsf, wg, peer)
            if rank == i % world:
                for _ in range(4):
                    spin = spin @ spin * 0 + 1          # this rank's consumer starts late
            sums.append(full.float().sum() + spin[0, 0] * 0)      # the consumer: reads the whole gathered output
            fulls_ok.append(torch.equal(full, wholes[i]))
        # one more step with every operand's scales in the reference's row layout: the kernel then loads the operands
        # with permuted rows and stores through rank-3 maps of the peers' buffers
        xr = ops.quantize(xs[0], 0, 1, sf_layout="ac4k")
        w4r, wsfr, wgr = parallel.quantize_weight_shard(w[lo:hi].contiguous(), None, "ac4k")
        full = parallel.column_parallel_linear_fused(xr[0], xr[1], xr[2], w4r, wsfr, wgr, peer)
        fulls_ok.append(torch.equal(full, wholes[0]))
        torch.cuda.synchronize()
        ok = all(fulls_ok) and all(float(sums[i]) == float(wholes[i].float().sum()) for i in range(steps))
        peer.close()
        assert ok, f"fused all-gather output differs from the single-GPU GEMM: {fulls_ok}"
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_parallel_gpus(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, 1024, 2048, 1024, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.kill()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
