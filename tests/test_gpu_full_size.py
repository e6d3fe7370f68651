"""The five target shapes at FULL size on the GPU.

The CPU oracle cannot finish these sizes in seconds, so each test combines
(a) the oracle on a sample of rows (rows are independent) with (b) properties that
hold for every row and are checked over the whole output with independent torch
arithmetic on the device: planted maxima and their columns, the unit mean square
of an RMSNorm, the zero mean / unit variance of a LayerNorm, the two orthogonality
relations of LayerNorm's dx (sum dx = 0 and sum dx * xhat = 0 when the statistics
are the row's own), and fp64 column sums for dgamma / dbeta.
Tolerances: argmax and max bit-exact; fp32 1e-5 relative (to the natural scale of
the quantity); bf16 2e-2.
"""
import pytest
import torch

from credit_b200 import _native as N
from credit_b200 import launchers as L
from credit_b200 import workloads as W
from oracle import reference_ops as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def launch(name, ins, **kw):
    outs = L.allocate_outputs(name, ins)
    L.NATIVE_LAUNCHERS[name](ins, outs, **kw)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    return outs


def sample_rows(rows):
    return torch.tensor(sorted({0, 1, rows // 3, rows // 2, rows - 2, rows - 1}))


def test_rmsnorm_forward_full(native_lib):
    rows, cols = 1024, 32768
    x, gamma = W.make_rmsnorm_inputs(rows, cols, DEV)
    (y,) = launch("rmsnorm_forward", (x, gamma))
    # property: mean square of y / gamma is 1 - eps / (ms + eps) for every row
    ms_out = (y.double() / gamma.double()).square().mean(-1)
    ms_in = x.double().square().mean(-1)
    assert torch.allclose(ms_out, ms_in / (ms_in + 1.0e-6), rtol=1e-5, atol=0)
    r = sample_rows(rows)
    want = O.rmsnorm_forward(x[r.to(DEV)].cpu(), gamma.cpu(), dtype=torch.float64)
    got = y[r.to(DEV)].cpu().double()
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)


def test_row_reduce_full(native_lib):
    rows, cols = 512, 1048576
    (x,) = W.make_row_reduce_inputs(rows, cols, DEV)
    s, m, a = launch("row_reduce", (x,))
    # the planted +10 is the unique maximum of its row: max and argmax are exact
    assert torch.equal(m, torch.full_like(m, 10.0))
    assert a.dtype == torch.int64
    assert torch.equal(x[torch.arange(rows, device=DEV), a], m)
    assert torch.equal(a, torch.argmax(x, dim=-1))
    want = x.double().sum(-1)
    scale = x.double().abs().sum(-1) / cols ** 0.5     # natural size of a sum of `cols` O(1) terms
    err = (s.double() - want).abs()
    assert bool((err <= 1e-5 * (want.abs() + scale)).all()), f"worst {float((err / (want.abs() + scale)).max()):.2e}"
    r = sample_rows(rows)
    ws, wm, wa = O.row_reduce(x[r.to(DEV)].cpu(), dtype=torch.float64)
    assert torch.equal(a[r.to(DEV)].cpu(), wa) and torch.equal(m[r.to(DEV)].cpu(), wm)


def test_layernorm_forward_full(native_lib):
    rows, cols = 4096, 131072
    x, gamma, beta = W.make_layernorm_forward_inputs(rows, cols, DEV)
    y, mean, rstd = launch("layernorm_forward", (x, gamma, beta))
    # statistics against fp64 on the device, row blocks to bound memory
    for r0 in range(0, rows, 512):
        xb = x[r0:r0 + 512].double()
        mu = xb.mean(-1)
        var = (xb - mu[:, None]).square().mean(-1)
        assert torch.allclose(mean[r0:r0 + 512].double(), mu, rtol=1e-5, atol=1e-5)
        assert torch.allclose(rstd[r0:r0 + 512].double(), torch.rsqrt(var + 1.0e-5), rtol=1e-5, atol=0)
        # property: (y - beta) / gamma has zero mean and unit variance (y is bf16: 2e-2)
        z = (y[r0:r0 + 512].double() - beta.double()) / gamma.double()
        assert bool((z.mean(-1).abs() < 2e-2).all())
        assert bool(((z.square().mean(-1) - 1.0).abs() < 2e-2).all())
    r = sample_rows(rows)
    wy, wm, wr = O.layernorm_forward(x[r.to(DEV)].cpu(), gamma.cpu(), beta.cpu(), dtype=torch.float64)
    got = y[r.to(DEV)].cpu().double()
    assert bool(((got - wy).abs() <= 2e-2 * wy.abs() + 1e-3 * wy.pow(2).mean(-1, keepdim=True).sqrt()).all())


def test_layernorm_backward_stats_full(native_lib):
    rows, cols = 8192, 65536
    x, dy, gamma, mean, rstd = W.make_layernorm_backward_stats_inputs(rows, cols, DEV)
    dx, dgamma, dbeta = launch("layernorm_backward_stats", (x, dy, gamma, mean, rstd))
    col_g = torch.zeros(cols, device=DEV, dtype=torch.float64)
    col_b = torch.zeros(cols, device=DEV, dtype=torch.float64)
    for r0 in range(0, rows, 512):
        sl = slice(r0, r0 + 512)
        xhat = (x[sl].double() - mean[sl].double()[:, None]) * rstd[sl].double()[:, None]
        dyb = dy[sl].double()
        col_g += (dyb * xhat).sum(0)
        col_b += dyb.sum(0)
        # orthogonality of dx (bf16 output: each element carries 2^-9 relative rounding)
        d = dx[sl].double()
        bound = 2e-2 * d.abs().sum(-1) / 16 + 1e-3
        assert bool((d.sum(-1).abs() <= bound).all())
        assert bool(((d * xhat).sum(-1).abs() <= bound * 4).all())
    scale = 4.0 * rows ** 0.5                  # natural size of a sum of `rows` O(1) terms
    assert bool(((dgamma.double() - col_g).abs() <= 1e-5 * col_g.abs() + 1e-5 * scale).all())
    assert bool(((dbeta.double() - col_b).abs() <= 1e-5 * col_b.abs() + 1e-5 * scale).all())
    r = sample_rows(rows).to(DEV)
    wdx, _, _ = O.layernorm_backward_stats(x[r].cpu(), dy[r].cpu(), gamma.cpu(), mean[r].cpu(), rstd[r].cpu(),
                                           dtype=torch.float64)
    got = dx[r].cpu().double()
    # relative 2e-2 per element plus an absolute term of 1e-3 of the ROW's own rms (dx of a row is a
    # difference of three terms of that size; the bf16 rounding of the result is 2^-9 of the element)
    row_rms = wdx.pow(2).mean(-1, keepdim=True).sqrt()
    assert bool(((got - wdx).abs() <= 2e-2 * wdx.abs() + 1e-3 * row_rms).all())


def test_layernorm_backward_is_linear_in_dy_full_width(native_lib):
    """dx(a * dy1 + dy2) = a * dx(dy1) + dx(dy2) at the full width (fp32 reference form)."""
    rows, cols = 64, 65536
    gen = torch.Generator(device=DEV).manual_seed(5)
    x = torch.empty(rows, cols, device=DEV).uniform_(-1, 1, generator=gen)
    d1 = torch.empty(rows, cols, device=DEV).uniform_(-1, 1, generator=gen)
    d2 = torch.empty(rows, cols, device=DEV).uniform_(-1, 1, generator=gen)
    gamma = torch.empty(cols, device=DEV).uniform_(0.75, 1.25, generator=gen)
    (a1,) = launch("layernorm_backward", (x, d1, gamma))
    (a2,) = launch("layernorm_backward", (x, d2, gamma))
    (a3,) = launch("layernorm_backward", (x, 0.5 * d1 + d2, gamma))
    assert torch.allclose(a3, 0.5 * a1 + a2, rtol=1e-4, atol=1e-5)
