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
