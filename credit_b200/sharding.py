"""Row-block sharding over the GPUs of one node.

Rows are independent in every workload of this library, so a matrix is split into
contiguous row blocks, one per rank (one process per GPU); gamma/beta/weights are
replicated and the outputs stay sharded. The single exchange step of the path is
LayerNorm backward's dgamma/dbeta, which are column sums over ALL rows: each rank
reduces its own rows, then one all-reduce over 2 * cols fp32 values finishes them.
The reference is single-GPU (device 0 is hard-coded, e.g.
`src/workloads/layernorm_backward.cu:443`); this module is new.

`torch.distributed` (NCCL on GPUs, gloo in CPU tests) carries the collective, or the
library's own one-kernel all-reduce over peer memory (`PeerGroup`); the finishing kernel
writes dgamma and dbeta into one contiguous [2, cols] buffer so that a single in-place
all-reduce on the compute stream follows it with no host synchronisation in between.
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
                                     opts=None, workspace: torch.Tensor | None = None, group=None,
                                     peer_group: "PeerGroup | None" = None) -> None:
    """LayerNorm backward on this rank's row block followed by the all-reduce of the
    parameter gradients. `inputs` = (x, dy, gamma, mean, rstd) of the local rows, `dx` the
    local output, `both` the buffer of `allocate_param_grads`. With `peer_group` the library's
    own peer-memory all-reduce runs instead of the process group's."""
    from .launchers import launch_layernorm_backward_stats

    launch_layernorm_backward_stats(inputs, (dx, both[0], both[1]), cluster_size, opts, workspace=workspace)
    if peer_group is not None:
        peer_group.allreduce(both)
    else:
        allreduce_param_grads(both, group)


class PeerGroup:
    """The library's own all-reduce of the [2, cols] buffer over peer memory
    (`credit_layernorm_bwd_allreduce_peer`: one kernel per rank, plain NVLink loads and stores,
    sums in rank order so that every rank gets identical bits). Each rank allocates a window,
    the 64-byte handles are gathered with `exchange` (default: `torch.distributed.all_gather_object`
    of the current process group, which may be gloo), and the peers' windows are mapped.

        group = PeerGroup(world, rank, max_cols)       # this rank's GPU is current
        group.allreduce(both)                          # collective, on the current stream
        group.close()                                  # after a host barrier
    """

    def __init__(self, world_size: int, rank: int, max_cols: int, exchange=None, connect: bool = True):
        import ctypes

        from . import _native as N

        self._lib = N.load()
        self._check = N.check
        self._handle_bytes = N.PEER_HANDLE_BYTES
        self._group = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(N.PEER_HANDLE_BYTES)
        N.check(self._lib.credit_peer_group_create(ctypes.byref(self._group), world_size, rank, max_cols, handle))
        self.world_size, self.rank, self.max_cols = world_size, rank, max_cols
        self.handle = handle.raw        # what the other ranks need of this one
        if connect and world_size > 1:
            if exchange is None:
                def exchange(mine: bytes) -> list[bytes]:
                    gathered: list = [None] * world_size
                    dist.all_gather_object(gathered, mine)
                    return gathered
            self.connect(exchange(self.handle))

    def connect(self, handles) -> None:
        """Maps the peers' windows; `handles` = one 64-byte handle per rank, in rank order. (A host that
        must survive a rank failing to create its window constructs with connect=False, agrees on
        the outcome over its own channel and calls this only when every rank has a handle.)"""
        import ctypes

        handles = list(handles)
        if len(handles) != self.world_size or any(len(h) != self._handle_bytes for h in handles):
            raise ValueError("expected one 64-byte handle per rank, in rank order")
        self._check(self._lib.credit_peer_group_connect(self._group, ctypes.create_string_buffer(b"".join(handles))))

    def allreduce(self, both: torch.Tensor) -> torch.Tensor:
        if both.dim() != 2 or both.shape[0] != 2 or both.dtype != torch.float32 or not both.is_contiguous():
            raise ValueError("expected the contiguous [2, cols] fp32 buffer of allocate_param_grads")
        self._check(self._lib.credit_layernorm_bwd_allreduce_peer(
            self._group, both.data_ptr(), both.shape[1], torch.cuda.current_stream(both.device).cuda_stream))
        return both

    def status(self) -> int:
        """0, or bit 0 set when a wait for a peer ran out (the buffer was then left unreduced)."""
        return int(self._lib.credit_peer_group_status(self._group))

    def close(self) -> None:
        if self._group:
            self._check(self._lib.credit_peer_group_destroy(self._group))
            self._group = None
