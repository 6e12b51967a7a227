"""Row-sharded multi-GPU execution of a GGUF linear layer.

Output rows are independent, so a weight `uint8 [N, rowbytes]` is split on dim 0 into `world` contiguous
slices of N/world rows - exactly the column-parallel slicing the reference's loader performs
(`load_column_parallel_weight`, vllm_gguf_plugin/quantization/params.py:230-247).  Activations are
replicated; every rank computes `[M, N/world]` and the slices are all-gathered along N.  The reference
has no collective of its own (the gather lives in vLLM's ColumnParallelLinear); here it is one
`all_gather_into_tensor` on the rank-major buffer `[world, M, N/world]` followed by a strided view.

One process per GPU (`torch.distributed`, backend "nccl" on GPUs; "gloo" works for the CPU tests with a
stand-in compute function).
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_rows(qweight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows [rank*N/world, (rank+1)*N/world) of a wire tensor (N must divide evenly)."""
    n = qweight.shape[0]
    if n % world:
        raise ValueError(f"N={n} is not divisible by the number of ranks {world}")
    per = n // world
    return qweight.narrow(0, rank * per, per)


def gather_columns(y_local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather `[M, N/world]` slices into `[M, N]` (rank r owns columns r*N/world ...)."""
    world = dist.get_world_size(group)
    m, per = y_local.shape
    if world == 1:
        return y_local
    buf = out if out is not None else torch.empty((world, m, per), dtype=y_local.dtype, device=y_local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(buf, y_local.contiguous(), group=group)
    else:  # gloo has no flat all-gather; a list of views into the same buffer is equivalent
        dist.all_gather([buf[r] for r in range(world)], y_local.contiguous(), group=group)
    return buf.permute(1, 0, 2).reshape(m, world * per)


class P2PGather:
    """All-gather of output slices by peer stores (kq_p2p_allgather) over buffers in torch symmetric memory.

    One instance owns `nbuf` gather buffers of `max_bytes * world` bytes each plus the flag arrays, all carved from
    one symmetric allocation; buffer b uses flag slot b.  `gather(y_local, b)` launches one kernel on the current
    stream and returns the local buffer viewed as [M, N] columns (rank r owns columns r*N/world ...).  Use a different
    buffer index for calls that may be in flight at the same time, and alternate two indices on one stream when the
    gathered data is read by later kernels.  Raises if symmetric memory cannot be set up (the caller then keeps
    the NCCL path)."""

    FLAG_BYTES_PER_SLOT = 8 * 4

    def __init__(self, max_bytes: int, nbuf: int, device: torch.device, group=None):
        import os
        # only plain peer loads/stores are used here: ask torch not to bind the allocation to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        from . import capi
        self._capi = capi
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("P2PGather supports at most 8 ranks")
        self.max_bytes = (max_bytes + 255) // 256 * 256
        self.nbuf = nbuf
        self.buf_bytes = self.max_bytes * self.world
        flag_bytes = (nbuf * self.FLAG_BYTES_PER_SLOT + 255) // 256 * 256
        total = flag_bytes + nbuf * self.buf_bytes
        self.mem = symm.empty((total,), dtype=torch.uint8, device=device)
        self.mem.zero_()
        torch.cuda.synchronize(device)
        self.hdl = symm.rendezvous(self.mem, group.group_name)
        self.hdl.barrier()                      # every rank's flags are zero before anyone publishes
        bases = [int(p) for p in self.hdl.buffer_ptrs]
        self.flag_ptrs = bases
        self.data_ptrs = [b + flag_bytes for b in bases]
        self.flag_bytes = flag_bytes
        self.epoch = torch.zeros(nbuf, dtype=torch.int32, device=device)
        self.done = torch.zeros(nbuf, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def gather(self, y_local: torch.Tensor, b: int) -> torch.Tensor:
        """Columns of all ranks as one [M, N] tensor (a copy out of the gather buffer)."""
        m, per = y_local.shape
        return self.gather_raw(y_local, b).permute(1, 0, 2).reshape(m, self.world * per)

    def gather_raw(self, y_local: torch.Tensor, b: int) -> torch.Tensor:
        """One kernel launch; returns the local gather buffer itself, viewed as [world, M, N/world]."""
        m, per = y_local.shape
        y_local = y_local.contiguous()
        nbytes = y_local.numel() * y_local.element_size()
        if nbytes > self.max_bytes or not 0 <= b < self.nbuf:
            raise ValueError(f"slice of {nbytes} bytes / buffer {b} outside what this P2PGather was sized for")
        dst = [p + b * self.buf_bytes for p in self.data_ptrs]
        self._capi.p2p_allgather(y_local, dst, self.flag_ptrs, self.epoch, self.done, b, self.rank, self.status)
        off = self.flag_bytes + b * self.buf_bytes
        return self.mem[off:off + self.world * nbytes].view(y_local.dtype).view(self.world, m, per)

    def check(self) -> None:
        """Synchronises; raises if any gather's bounded wait for a peer ran out."""
        st = int(self.status.item())
        if st:
            raise RuntimeError(f"kq_p2p_allgather: wait for rank {st - 1} timed out")


class ShardedGGUFLinear:
    """One rank's slice of a row-sharded layer plus the gather."""

    def __init__(self, qweight_local: torch.Tensor, qweight_type: int,
                 matmul: Callable[[torch.Tensor, torch.Tensor, int], torch.Tensor], group=None):
        self.qweight = qweight_local
        self.qweight_type = qweight_type
        self.matmul = matmul
        self.group = group

    @classmethod
    def from_full(cls, qweight: torch.Tensor, qweight_type: int, matmul, group=None):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        return cls(shard_rows(qweight, rank, world).contiguous(), qweight_type, matmul, group)

    def local(self, x: torch.Tensor) -> torch.Tensor:
        return self.matmul(x, self.qweight, self.qweight_type)

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        return gather_columns(self.local(x), self.group)
