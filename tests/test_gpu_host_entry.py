"""The host-buffer entry points (`credit_*_host`): data in host memory, streamed through device
scratch in row blocks. Results must agree with those of the device-pointer entry points on the
same inputs: index and maximum outputs exactly, floating outputs to rounding (a block has fewer
rows than the matrix, so the planner may pick another cluster size and with it another order of
the fp32 additions: 1e-5 relative for fp32, one bf16 ulp for bf16), with minimal scratch (many
blocks) and with ample scratch (one block), from pinned and from pageable memory."""
import pytest
import torch

from credit_b200 import _native as N
from credit_b200 import host as H
from credit_b200 import launchers as L
from credit_b200 import workloads as W

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def device_result(name, inputs):
    ins = tuple(t.to(DEV) for t in inputs)
    outs = L.allocate_outputs(name, ins)
    L.NATIVE_LAUNCHERS[name](ins, outs)
    torch.cuda.synchronize()
    return tuple(o.cpu() for o in outs)


def scratch_for(name, rows, cols, dtype, extra=0, hidden=0):
    return torch.empty(H.scratch_bytes(name, rows, cols, dtype, hidden) + extra, dtype=torch.uint8, device=DEV)


def same(got, want, what=""):
    """Equal up to the order of fp32 additions."""
    if got.dtype == torch.bfloat16:
        torch.testing.assert_close(got.float(), want.float(), rtol=2.0 ** -7, atol=2.0 ** -7, msg=what or None)
    else:
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6, msg=what or None)


def maybe_pin(tensors, pin):
    return tuple(t.pin_memory() for t in tensors) if pin else tensors


@pytest.fixture(autouse=True)
def _healthy(native_lib):
    yield
    assert N.device_status() == 0


@pytest.mark.parametrize("pin", [True, False])
@pytest.mark.parametrize("rows,cols,extra", [(300, 262144, 0), (300, 262144, 1 << 30), (5, 1000, 0)])
def test_row_reduce_host(rows, cols, extra, pin):
    (x,) = maybe_pin(W.make_row_reduce_inputs(rows, cols, "cpu", seed=2), pin)
    want = device_result("row_reduce", (x,))
    s, m, a = torch.empty(rows), torch.empty(rows), torch.empty(rows, dtype=torch.int64)
    H.row_reduce(x, s, m, a, scratch_for("row_reduce", rows, cols, torch.float32, extra))
    assert torch.equal(a, want[2]) and torch.equal(m, want[1])
    torch.testing.assert_close(s, want[0], rtol=1e-5, atol=1e-5 * cols ** 0.5)


@pytest.mark.parametrize("rows,cols,dtype,extra", [(2100, 32768, torch.float32, 0), (2100, 32768, torch.float32, 1 << 30),
                                                   (700, 4096, torch.bfloat16, 0), (9, 1000, torch.float32, 0)])
def test_rmsnorm_forward_host(rows, cols, dtype, extra):
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=3)
    x = x.to(dtype).pin_memory()
    (want,) = device_result("rmsnorm_forward", (x, gamma))
    y = torch.full_like(x, float("nan")).pin_memory()
    H.rmsnorm_forward(x, gamma, y, scratch_for("rmsnorm_forward", rows, cols, dtype, extra))
    same(y, want)


@pytest.mark.parametrize("rows,cols,extra", [(600, 131072, 0), (600, 131072, 1 << 30), (33, 4099, 0)])
def test_layernorm_forward_host(rows, cols, extra):
    inputs = W.make_layernorm_forward_inputs(rows, cols, "cpu", seed=4)
    want = device_result("layernorm_forward", inputs)
    x, gamma, beta = inputs
    y = torch.full_like(x, float("nan")).pin_memory()
    mean, rstd = torch.empty(rows), torch.empty(rows)
    H.layernorm_forward(x.pin_memory(), gamma, beta, y, mean, rstd,
                        scratch_for("layernorm_forward", rows, cols, x.dtype, extra))
    same(y, want[0], "y")
    torch.testing.assert_close(mean, want[1], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(rstd, want[2], rtol=1e-5, atol=0.0)


@pytest.mark.parametrize("rows,cols,dtype,extra", [(1000, 65536, torch.bfloat16, 0), (1000, 65536, torch.bfloat16, 1 << 30),
                                                   (70, 1000, torch.float32, 0)])
def test_layernorm_backward_stats_host(rows, cols, dtype, extra):
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=5, dtype=dtype)
    want_dx, want_dg, want_db = device_result("layernorm_backward_stats", inputs)
    x, dy, gamma, mean, rstd = inputs
    dx = torch.full_like(x, float("nan")).pin_memory()
    dgamma, dbeta = torch.full((cols,), float("nan")), torch.full((cols,), float("nan"))
    H.layernorm_backward_stats(x.pin_memory(), dy.pin_memory(), gamma, mean, rstd, dx, dgamma, dbeta,
                               scratch_for("layernorm_backward_stats", rows, cols, dtype, extra))
    same(dx, want_dx, "dx")
    # column sums: the blocks change the order of the fp32 additions
    scale = 4.0 * rows ** 0.5
    assert bool(((dgamma - want_dg).abs() <= 1e-5 * want_dg.abs() + 1e-5 * scale).all())
    assert bool(((dbeta - want_db).abs() <= 1e-5 * want_db.abs() + 1e-5 * scale).all())


def test_ffn_forward_host():
    m, d, h = 256, 512, 1024
    x, w1, w2, gamma = W.make_ffn_inputs(m, d, "cpu", seed=6, hidden=h)
    w1p, w2p, gd = L.pack_ffn_weight(w1.to(DEV)), L.pack_ffn_weight(w2.to(DEV)), gamma.to(DEV)
    want = torch.empty_like(x, device=DEV)
    L.launch_ffn_forward((x.to(DEV), w1p, w2p, gd), (want,))
    torch.cuda.synchronize()
    y = torch.full_like(x, float("nan")).pin_memory()
    H.ffn_forward(x.pin_memory(), w1p, w2p, gd, y, scratch_for("ffn_forward", m, d, torch.bfloat16, hidden=h))
    assert torch.equal(y, want.cpu())


def test_host_calls_reject_bad_scratch():
    rows, cols = 16, 4096
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=1)
    y = torch.empty_like(x)
    small = torch.empty(1024, dtype=torch.uint8, device=DEV)
    with pytest.raises(N.CreditError) as err:
        H.rmsnorm_forward(x, gamma, y, small)
    assert err.value.code == N.ERR_WORKSPACE
    with pytest.raises(ValueError):
        H.rmsnorm_forward(x.to(DEV), gamma, y, small)      # device tensor where host memory is expected
