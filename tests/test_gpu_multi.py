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


def _abi_worker(rank: int, world: int, id_path: str, rows: int, cols: int, out):
    """The same sharded call with the collective of the C ABI (credit_comm_*,
    credit_layernorm_bwd_allreduce) instead of torch.distributed: the id travels through a file."""
    import ctypes
    import time
    from pathlib import Path

    from credit_b200 import _native as N
    from credit_b200 import launchers as L
    from credit_b200 import sharding
    from credit_b200 import workloads as W
    from oracle import reference_ops as O

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    lib = N.load()
    ident = ctypes.create_string_buffer(128)
    path = Path(id_path)
    if rank == 0:
        N.check(lib.credit_comm_get_unique_id(ident))
        tmp = path.with_suffix(".tmp")
        tmp.write_bytes(ident.raw)
        tmp.rename(path)
    else:
        deadline = time.time() + 60
        while not path.exists():
            if time.time() > deadline:
                raise RuntimeError("rank 0 never published the id")
            time.sleep(0.05)
        ident = ctypes.create_string_buffer(path.read_bytes(), 128)
    comm = ctypes.c_void_p()
    N.check(lib.credit_comm_init_rank(ctypes.byref(comm), world, rank, ident))
    try:
        full = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=9)
        x, dy, gamma, mean, rstd = full
        r0, r1 = sharding.shard_rows(rows, world, rank)
        local = (x[r0:r1].to(dev), dy[r0:r1].to(dev), gamma.to(dev), mean[r0:r1].to(dev), rstd[r0:r1].to(dev))
        dx = torch.empty_like(local[0])
        both, dgamma, dbeta = sharding.allocate_param_grads(cols, dev)
        stream = torch.cuda.current_stream().cuda_stream
        L.launch_layernorm_backward_stats(local, (dx, dgamma, dbeta))
        N.check(lib.credit_layernorm_bwd_allreduce(comm, both.data_ptr(), cols, stream))
        torch.cuda.synchronize()
        want_dx, want_dg, want_db = O.layernorm_backward_stats(*full, dtype=torch.float64)

        def close(got, want, rtol, scale):
            err = (got.double().cpu() - want).abs()
            return bool((err <= rtol * want.abs() + rtol * scale).all())

        out[rank] = (close(dx, want_dx[r0:r1], 2e-2, 2.0) and close(dgamma, want_dg, 1e-5, 4.0 * rows ** 0.5)
                     and close(dbeta, want_db, 1e-5, 4.0 * rows ** 0.5) and N.device_status() == 0)
    finally:
        N.check(lib.credit_comm_destroy(comm))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_c_abi_collective_allreduces_parameter_gradients(native_lib, tmp_path):
    import torch.multiprocessing as mp

    world, rows, cols = 2, 301, 4096
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_abi_worker, args=(world, str(tmp_path / "nccl_id.bin"), rows, cols, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_c_abi_collective_in_a_world_of_one(native_lib):
    """One rank: init, an all-reduce that is the identity, destroy; bad arguments are reported."""
    import ctypes

    from credit_b200 import _native as N

    lib = N.load()
    torch.cuda.set_device(0)
    ident = ctypes.create_string_buffer(128)
    N.check(lib.credit_comm_get_unique_id(ident))
    comm = ctypes.c_void_p()
    N.check(lib.credit_comm_init_rank(ctypes.byref(comm), 1, 0, ident))
    buf = torch.arange(2 * 1000, dtype=torch.float32, device="cuda:0").reshape(2, 1000)
    want = buf.clone()
    N.check(lib.credit_layernorm_bwd_allreduce(comm, buf.data_ptr(), 1000, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(buf, want)
    assert lib.credit_layernorm_bwd_allreduce(comm, None, 1000, None) == N.ERR_INVALID_ARGUMENT
    assert lib.credit_layernorm_bwd_allreduce(None, buf.data_ptr(), 1000, None) == N.ERR_INVALID_ARGUMENT
    assert lib.credit_comm_init_rank(ctypes.byref(ctypes.c_void_p()), 2, 5, ident) == N.ERR_INVALID_ARGUMENT
    N.check(lib.credit_comm_destroy(comm))


def _peer_worker(rank: int, world: int, port: int, rows: int, cols: int, out):
    """The sharded call with the library's own all-reduce over peer memory (one kernel per rank, CUDA
    IPC windows); the handles travel through a gloo process group. Several calls in a row, so both
    data buffers and several epochs are used; an odd width takes the scalar path."""
    import torch.distributed as dist

    from credit_b200 import _native as N
    from credit_b200 import sharding
    from credit_b200 import workloads as W
    from oracle import reference_ops as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    peers = None
    try:
        peers = sharding.PeerGroup(world, rank, max_cols=cols)
        full = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=9)
        x, dy, gamma, mean, rstd = full
        r0, r1 = sharding.shard_rows(rows, world, rank)
        local = (x[r0:r1].to(dev), dy[r0:r1].to(dev), gamma.to(dev), mean[r0:r1].to(dev), rstd[r0:r1].to(dev))
        dx = torch.empty_like(local[0])
        both, dgamma, dbeta = sharding.allocate_param_grads(cols, dev)
        want_dx, want_dg, want_db = O.layernorm_backward_stats(*full, dtype=torch.float64)

        def close(got, want, rtol, scale):
            err = (got.double().cpu() - want).abs()
            return bool((err <= rtol * want.abs() + rtol * scale).all())

        ok = True
        results = []
        for _ in range(5):
            sharding.layernorm_backward_stats_sharded(local, dx, both, peer_group=peers)
            torch.cuda.synchronize()
            ok = ok and close(dgamma, want_dg, 1e-5, 4.0 * rows ** 0.5) and close(dbeta, want_db, 1e-5, 4.0 * rows ** 0.5)
            results.append(both.cpu().clone())
        ok = ok and close(dx, want_dx[r0:r1], 2e-2, 2.0)
        # a plain vector of odd length (scalar path): every rank contributes rank + 1
        odd = torch.full((2, 333), float(rank + 1), device=dev)
        peers.allreduce(odd)
        torch.cuda.synchronize()
        ok = ok and bool((odd == world * (world + 1) / 2).all())
        ok = ok and peers.status() == 0 and N.device_status() == 0
        # the sums are added in rank order on every rank: identical bits everywhere
        gathered = [None] * world
        dist.all_gather_object(gathered, results[-1].numpy().tobytes())
        ok = ok and all(g == gathered[0] for g in gathered)
        out[rank] = ok
        dist.barrier()      # nobody closes a window a peer may still read
    finally:
        if peers is not None:
            peers.close()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_allreduce_of_parameter_gradients(native_lib):
    import torch.multiprocessing as mp

    world, rows, cols = 2, 301, 4096
    port = _free_port()
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_peer_worker, args=(world, port, rows, cols, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_peer_group_in_a_world_of_one(native_lib):
    """One rank: the all-reduce is the identity and needs no peers; bad arguments are reported."""
    import ctypes

    from credit_b200 import _native as N
    from credit_b200 import sharding

    torch.cuda.set_device(0)
    group = sharding.PeerGroup(1, 0, max_cols=1000)
    buf = torch.arange(2 * 1000, dtype=torch.float32, device="cuda:0").reshape(2, 1000)
    want = buf.clone()
    group.allreduce(buf)
    torch.cuda.synchronize()
    assert torch.equal(buf, want) and group.status() == 0
    with pytest.raises(N.CreditError):
        group.allreduce(torch.zeros(2, 1001, device="cuda:0"))      # wider than the group's windows
    group.close()
    lib = N.load()
    handle = ctypes.create_string_buffer(N.PEER_HANDLE_BYTES)
    assert lib.credit_peer_group_create(ctypes.byref(ctypes.c_void_p()), 17, 0, 1000, handle) == N.ERR_INVALID_ARGUMENT
    assert lib.credit_peer_group_create(ctypes.byref(ctypes.c_void_p()), 2, 2, 1000, handle) == N.ERR_INVALID_ARGUMENT
    assert lib.credit_layernorm_bwd_allreduce_peer(None, buf.data_ptr(), 1000, None) == N.ERR_INVALID_ARGUMENT


def _peer_timeout_worker(rank: int, world: int, port: int, out):
    """Only rank 0 calls the all-reduce: its bounded wait for rank 1's flag runs out (about a second),
    the kernel returns, the group's status word says so and the buffer is left as it was. No GPU
    faults or hangs: the wait is a polling loop with a time limit."""
    import torch.distributed as dist

    from credit_b200 import sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    peers = None
    try:
        peers = sharding.PeerGroup(world, rank, max_cols=1024)
        ok = peers.status() == 0
        if rank == 0:
            buf = torch.arange(2 * 1024, dtype=torch.float32, device=dev).reshape(2, 1024)
            want = buf.clone()
            peers.allreduce(buf)
            torch.cuda.synchronize()          # returns after the wait has run out
            ok = ok and peers.status() == 1 and torch.equal(buf, want)
            # the context is still usable
            ok = ok and float((buf + 1).sum().item()) == float(want.sum().item()) + buf.numel()
        out[rank] = ok
        dist.barrier()
    finally:
        if peers is not None:
            peers.close()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_allreduce_wait_is_bounded(native_lib):
    import torch.multiprocessing as mp

    world = 2
    port = _free_port()
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_peer_timeout_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}
