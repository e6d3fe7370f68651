"""Two ranks, one GPU each, NCCL: rows sharded, dgamma/dbeta all-reduced.
Skipped when fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, rows: int, cols: int, out):
    import torch.distributed as dist

    from credit_b200 import _native as N
    from credit_b200 import sharding
    from credit_b200 import workloads as W
    from oracle import reference_ops as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        full = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=9)
        x, dy, gamma, mean, rstd = full
        r0, r1 = sharding.shard_rows(rows, world, rank)
        local = (x[r0:r1].to(dev), dy[r0:r1].to(dev), gamma.to(dev), mean[r0:r1].to(dev), rstd[r0:r1].to(dev))
        dx = torch.empty_like(local[0])
        both, dgamma, dbeta = sharding.allocate_param_grads(cols, dev)
        sharding.layernorm_backward_stats_sharded(local, dx, both, cluster_size=4)
        torch.cuda.synchronize()
        want_dx, want_dg, want_db = O.layernorm_backward_stats(*full, dtype=torch.float64)

        def close(got, want, rtol, scale):
            err = (got.double().cpu() - want).abs()
            return bool((err <= rtol * want.abs() + rtol * scale).all())

        ok = (close(dx, want_dx[r0:r1], 2e-2, 2.0) and close(dgamma, want_dg, 1e-5, 4.0 * rows ** 0.5)
              and close(dbeta, want_db, 1e-5, 4.0 * rows ** 0.5) and N.device_status() == 0)
        out[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_layernorm_backward_allreduces_parameter_gradients(native_lib):
    import torch.multiprocessing as mp

    world, rows, cols = 2, 301, 4096
    port = _free_port()
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_worker, args=(world, port, rows, cols, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}
