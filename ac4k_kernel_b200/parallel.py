"""Column-parallel NVFP4 linear over the GPUs of one node (one process per GPU).

The reference has no multi-GPU code; this module defines the variant the B200 build adds:
the weight [N, K] is split by rows (output columns) over the ranks, activations are
replicated, every rank computes D[:, r*N/w : (r+1)*N/w] with the single-GPU kernel and the
bf16 outputs are all-gathered over NVLink with NCCL.  For the result to equal the single-GPU
result bit for bit, every shard must be quantised with the global scale of the WHOLE weight:
the per-shard amax scales are combined with one all-reduce(max) of a single float (exact and
order independent).

Only the collective plumbing lives here; it works with any torch.distributed backend, which is
how the CPU tests exercise it (gloo, world size 2).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(n: int, rank: int, world: int, align: int = 128):
    """Rows [lo, hi) of the weight owned by `rank`.  N must split into `world` equal parts that
    are multiples of `align` (128 keeps every shard on whole 128-row scale tiles)."""
    if n % world != 0 or (n // world) % align != 0:
        raise ValueError(f"N={n} does not split into {world} shards of a multiple of {align} rows")
    per = n // world
    return rank * per, (rank + 1) * per


def allreduce_max_scale(local_scale: torch.Tensor, group=None) -> torch.Tensor:
    """max over ranks of a 0-dim fp32 scale, in place.  amax/max_scale is monotonic in amax, so
    the max of the per-shard global scales is the global scale of the whole tensor."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(local_scale, op=dist.ReduceOp.MAX, group=group)
    return local_scale


def quantize_weight_shard(w_shard: torch.Tensor, group=None, sf_layout: str = "128x4"):
    """Quantise this rank's rows of the weight with the whole-tensor global scale.
    Returns (packed, scales, global_scale) like `ops.quantize`."""
    from .ops.quant import _global_scale, quantize_nvfp4, FLOAT4_E2M1_MAX, FLOAT8_E4M3_MAX
    from .ops.utils import align_up, ceil_div
    g = _global_scale(w_shard, FLOAT4_E2M1_MAX * FLOAT8_E4M3_MAX)
    allreduce_max_scale(g, group)
    n, k = w_shard.shape
    kp = align_up(k, 64)
    out = torch.empty((n, kp // 2), dtype=torch.uint8, device=w_shard.device)
    if sf_layout == "ac4k":
        sf_shape = (kp // 64, align_up(n, 16), 4)
    else:
        sf_shape = (ceil_div(n, 128), kp // 64, 32, 4, 4)
    sf = torch.empty(sf_shape, dtype=torch.float8_e4m3fn, device=w_shard.device)
    quantize_nvfp4(out, sf, w_shard, g, 0, 1, False)
    return out, sf, g


def gather_columns(local_out: torch.Tensor, gathered: torch.Tensor | None = None, group=None):
    """All-gather the [M, N/w] outputs of all ranks into a [w, M, N/w] tensor (rank-major slabs,
    the layout NCCL writes without an extra pass).  `columns_view` gives the [M, N] ordering."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    m, ns = local_out.shape
    if gathered is None:
        gathered = torch.empty((world, m, ns), dtype=local_out.dtype, device=local_out.device)
    if world == 1:
        gathered[0].copy_(local_out)
    else:
        dist.all_gather_into_tensor(gathered.view(world * m, ns), local_out.contiguous(), group=group)
    return gathered


def columns_view(gathered: torch.Tensor) -> torch.Tensor:
    """[w, M, N/w] -> [M, N] (a strided view; call .contiguous() for row-major memory)."""
    w, m, ns = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, w * ns)


def column_parallel_linear(x, x_scale, x_global_scale, w_shard, w_shard_scale, w_global_scale,
                           bias_shard=None, local_out=None, gathered=None, group=None):
    """One step of the column-parallel layer: local NVFP4 GEMM on this rank's shard, then the
    all-gather of the bf16 output.  Returns (gathered [w, M, N/w], local_out)."""
    from .ops.linear import linear
    local_out = linear(x, x_scale, x_global_scale, w_shard, w_shard_scale, w_global_scale,
                       bias=bias_shard, out=local_out)
    return gather_columns(local_out, gathered, group), local_out


def column_parallel_linear_pipelined(x, x_scale, x_global_scale, w_shard, w_shard_scale, w_global_scale,
                                     gathered, bias_shard=None, chunks=4, group=None, comm_stream=None):
    """Column-parallel step with the exchange overlapped with the GEMM.

    The M rows are cut into `chunks` blocks (multiples of 128 rows, so 128x4 scale tiles slice
    cleanly).  Block i is computed straight into this rank's slab of `gathered` ([w, M, N/w]) and
    then sent to every peer with grouped NCCL send/recv on `comm_stream` while block i+1 is being
    computed.  Results are identical to `column_parallel_linear`.  Returns `gathered`; the caller
    must wait on `comm_stream` (the function leaves the current stream waiting on it).
    """
    from .ops.linear import linear
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    m = x.shape[0]
    if x_scale.dim() != 5:
        raise ValueError("the pipelined variant slices activations by 128-row scale tiles (sf_layout='128x4')")
    per = -(-m // chunks)
    per = -(-per // 128) * 128
    main = torch.cuda.current_stream()
    if comm_stream is None:
        comm_stream = torch.cuda.Stream()
    for r0 in range(0, m, per):
        r1 = min(m, r0 + per)
        out_view = gathered[rank, r0:r1]
        linear(x[r0:r1], x_scale[r0 // 128:-(-r1 // 128)], x_global_scale, w_shard, w_shard_scale,
               w_global_scale, bias=bias_shard, out=out_view)
        if world > 1:
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(comm_stream):
                comm_stream.wait_event(ready)
                ops = []
                for peer in range(world):
                    if peer == rank:
                        continue
                    ops.append(dist.P2POp(dist.isend, out_view, peer, group))
                    ops.append(dist.P2POp(dist.irecv, gathered[peer, r0:r1], peer, group))
                for req in dist.batch_isend_irecv(ops):
                    req.wait()
    main.wait_stream(comm_stream)
    return gathered


class PeerOutput:
    """The gathered output [M, N] (row-major, whole matrix) of the column-parallel layer, one copy
    per rank, every copy mapped into every rank's process so that a GEMM epilogue can store its
    tiles to all of them over NVLink.

    `nbuf` copies are kept per rank (default 2) and used in turn, one per step.  With a single copy a
    rank that is ahead could start storing step i+1 into a peer's buffer while that peer's kernels still
    read step i from it: the one-element all-reduce that closes a step orders every rank's reads of step
    i after every rank's stores of step i, but nothing orders the stores of step i+1 after those reads.
    With two copies, step i+2 reuses the buffer of step i, and a rank can only reach step i+2 after the
    all-reduce of step i+1, which every rank enqueues behind its own readers of step i.

    The memory comes from the library's `ac4k_peer_alloc` (plain cudaMalloc + CUDA IPC handle); the
    handles travel through `all_gather_object` of the process group.  `tensor` is this rank's copy of
    the step last computed, as a torch tensor; `ptrs[i]` is the device address, in this process, of rank
    i's first copy.  Call `close()` (collective) before the process group is destroyed.
    """

    def __init__(self, m: int, n: int, dtype=torch.bfloat16, group=None, nbuf: int = 2):
        import ctypes
        from ._lib import LIB, check
        if not dist.is_initialized():
            raise RuntimeError("PeerOutput needs an initialised process group")
        if nbuf < 1:
            raise ValueError("nbuf must be at least 1")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.m, self.n, self.dtype, self.nbuf = m, n, dtype, nbuf
        self.buf_bytes = m * n * torch.empty((), dtype=dtype).element_size()
        self.buf_bytes = -(-self.buf_bytes // 256) * 256
        self.step = 0
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        check(LIB.ac4k_peer_alloc(self.buf_bytes * nbuf, ctypes.byref(ptr), handle), "ac4k_peer_alloc")
        self._own = ptr.value
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self._own)
                continue
            q = ctypes.c_void_p()
            check(LIB.ac4k_peer_open(h, ctypes.byref(q)), f"ac4k_peer_open(rank {r})")
            self.ptrs.append(q.value)
        # this rank's copies as tensors (CUDA array interface: no copy, this object keeps them alive)
        typestr = {torch.bfloat16: "<i2", torch.float16: "<f2"}[dtype]
        self._holders, self.tensors = [], []
        for b in range(nbuf):
            holder = type("_Mem", (), {})()
            holder.__cuda_array_interface__ = {"shape": (m, n), "typestr": typestr,
                                               "data": (self._own + b * self.buf_bytes, False),
                                               "version": 3, "strides": None}
            t = torch.as_tensor(holder, device=torch.device("cuda", torch.cuda.current_device()))
            self.tensors.append(t.view(dtype) if t.dtype != dtype else t)
            self._holders.append(holder)

    @property
    def tensor(self):
        """This rank's copy of the step computed last (the first copy before any step)."""
        return self.tensors[(self.step - 1) % self.nbuf if self.step else 0]

    def destinations(self, buf: int = 0):
        """Device addresses of copy `buf`, ordered for this rank: own copy first, then the peers starting
        with the next rank, so that at any moment different ranks are storing to different peers."""
        return [self.ptrs[(self.rank + i) % self.world] + buf * self.buf_bytes for i in range(self.world)]

    def close(self):
        from ._lib import LIB, check
        torch.cuda.synchronize()
        dist.barrier(group=self.group)              # nobody is still storing into a peer
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p is not None:
                check(LIB.ac4k_peer_close(p), "ac4k_peer_close")
        self.ptrs = []
        dist.barrier(group=self.group)              # every mapping is closed before the owners free
        self.tensors = []
        if self._own is not None:
            check(LIB.ac4k_peer_free(self._own), "ac4k_peer_free")
            self._own = None


def column_parallel_linear_fused(x, x_scale, x_global_scale, w_shard, w_shard_scale, w_global_scale,
                                 peer_out: PeerOutput, bias_shard=None, sync: torch.Tensor | None = None):
    """Column-parallel step with the all-gather fused into the GEMM epilogue: this rank's kernel
    stores each finished tile of its [M, N/w] columns into every rank's [M, N] buffer (TMA stores; the
    peers' buffers are reached over NVLink).  A one-element all-reduce on the same stream then orders
    every rank's reads after every rank's stores.  Consecutive steps use the copies of `peer_out` in
    turn (see PeerOutput).  Returns this rank's full [M, N] output of this step, valid on the current
    stream after the call and until `nbuf` further steps have been issued."""
    from . import _cuda_ops
    lo, _ = shard_bounds(peer_out.n, peer_out.rank, peer_out.world, align=8)
    buf = peer_out.step % peer_out.nbuf
    out = peer_out.tensors[buf]
    _cuda_ops.linear_nvfp4_gather(peer_out.destinations(buf), peer_out.n, lo, out, x, x_scale,
                                  x_global_scale, w_shard, w_shard_scale, w_global_scale, bias_shard)
    peer_out.step += 1
    if peer_out.world > 1:
        if sync is None:
            sync = torch.zeros(1, dtype=torch.float32, device=x.device)
        dist.all_reduce(sync, group=peer_out.group)
    return out
