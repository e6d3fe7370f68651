"""Row sharding and the dgamma/dbeta all-reduce with two gloo ranks on the CPU.

The kernels need a GPU, so each rank computes its local column sums with the CPU
oracle; what is under test is the host-side logic: the row partition and the
in-place all-reduce of the [2, cols] buffer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from credit_b200 import sharding
from credit_b200 import workloads as W
from oracle import reference_ops as O


@pytest.mark.parametrize("rows,world", [(10, 1), (10, 3), (7, 8), (0, 4), (8192, 8)])
def test_shard_rows_tiles_the_matrix(rows, world):
    blocks = [sharding.shard_rows(rows, world, r) for r in range(world)]
    assert blocks[0][0] == 0 and blocks[-1][1] == rows
    for (a0, a1), (b0, b1) in zip(blocks, blocks[1:]):
        assert a1 == b0
    sizes = [b - a for a, b in blocks]
    assert max(sizes) - min(sizes) <= 1


def test_shard_rows_rejects_bad_ranks():
    with pytest.raises(ValueError):
        sharding.shard_rows(4, 2, 2)
    with pytest.raises(ValueError):
        sharding.shard_rows(-1, 2, 0)


def test_allreduce_is_a_no_op_without_a_process_group():
    both, dg, db = sharding.allocate_param_grads(8, "cpu")
    both.fill_(3.0)
    assert sharding.allreduce_param_grads(both) is both
    assert float(dg.sum()) == 24.0 and db.data_ptr() == both[1].data_ptr()
    with pytest.raises(ValueError):
        sharding.allreduce_param_grads(torch.zeros(3, 8))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, rows: int, cols: int, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, dy, gamma, mean, rstd = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=3,
                                                                          dtype=torch.float32)
        r0, r1 = sharding.shard_rows(rows, world, rank)
        _, dg, db = O.layernorm_backward_stats(x[r0:r1], dy[r0:r1], gamma, mean[r0:r1], rstd[r0:r1])
        both, dgamma, dbeta = sharding.allocate_param_grads(cols, "cpu")
        dgamma.copy_(dg)
        dbeta.copy_(db)
        sharding.allreduce_param_grads(both)
        _, want_dg, want_db = O.layernorm_backward_stats(x, dy, gamma, mean, rstd)
        ok = torch.allclose(dgamma, want_dg, rtol=1e-5, atol=1e-5) and torch.allclose(dbeta, want_db, rtol=1e-5, atol=1e-5)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_ranks_allreduce_matches_the_unsharded_column_sums():
    world, rows, cols = 2, 37, 96
    port = _free_port()
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_worker, args=(world, port, rows, cols, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}
