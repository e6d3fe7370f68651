"""Row-block sharding over the GPUs of one node.

Rows are independent in every workload of this library, so a matrix is split into
contiguous row blocks, one per rank (one process per GPU); gamma/beta/weights are
replicated and the outputs stay sharded. The single exchange step of the path is
LayerNorm backward's dgamma/dbeta, which are column sums over ALL rows: each rank
reduces its own rows, then one all-reduce over 2 * cols fp32 values finishes them.
The reference is single-GPU (device 0 is hard-coded, e.g.
`src/workloads/layernorm_backward.cu:443`); this module is new.

`torch.distributed` (NCCL on GPUs, gloo in CPU tests) carries the collective; the
finishing kernel writes dgamma and dbeta into one contiguous [2, cols] buffer so
that a single in-place all-reduce on the compute stream follows it with no host
synchronisation in between.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the row block of `rank`: sizes differ by at most one row and
    the blocks tile [0, rows) in rank order."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of size {world_size}")
    if rows < 0:
        raise ValueError("rows must be non-negative")
    base, extra = divmod(rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def allocate_param_grads(cols: int, device) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One [2, cols] fp32 buffer and its two rows (dgamma, dbeta) as views."""
    both = torch.empty((2, cols), dtype=torch.float32, device=device)
    return both, both[0], both[1]


def allreduce_param_grads(both: torch.Tensor, group=None) -> torch.Tensor:
    """Sums the [2, cols] dgamma/dbeta buffer over all ranks, in place, on the current
    stream. A no-op outside a process group or in a world of one."""
    if both.dim() != 2 or both.shape[0] != 2 or both.dtype != torch.float32:
        raise ValueError("expected the [2, cols] fp32 buffer of allocate_param_grads")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(both, op=dist.ReduceOp.SUM, group=group)
    return both


def layernorm_backward_stats_sharded(inputs, dx: torch.Tensor, both: torch.Tensor, cluster_size: int = 0,
                                     opts=None, workspace: torch.Tensor | None = None, group=None) -> None:
    """LayerNorm backward on this rank's row block followed by the all-reduce of the
    parameter gradients. `inputs` = (x, dy, gamma, mean, rstd) of the local rows, `dx` the
    local output, `both` the buffer of `allocate_param_grads`."""
    from .launchers import launch_layernorm_backward_stats

    launch_layernorm_backward_stats(inputs, (dx, both[0], both[1]), cluster_size, opts, workspace=workspace)
    allreduce_param_grads(both, group)
