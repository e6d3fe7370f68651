"""The CPU oracle against the reference's own outputs (golden vectors) and
against itself in fp64."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import reference_ops as O

GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_workloads.npz"


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def _cases(golden, name):
    keys = sorted({k.rsplit("/", 1)[0] for k in golden.files if k.startswith(name + "/") and "x" in k.split("/")[1]})
    for key in keys:
        ins, outs = [], []
        i = 0
        while f"{key}/in{i}" in golden.files:
            ins.append(torch.from_numpy(golden[f"{key}/in{i}"]))
            i += 1
        i = 0
        while f"{key}/out{i}" in golden.files:
            outs.append(torch.from_numpy(golden[f"{key}/out{i}"]))
            i += 1
        yield key, ins, outs


@pytest.mark.parametrize("name", sorted(O.REFERENCE_FUNCTIONS))
def test_restatement_matches_reference_outputs(golden, name):
    """Every restated function reproduces what the reference's function returned."""
    seen = 0
    for key, ins, outs in _cases(golden, name):
        got = O.REFERENCE_FUNCTIONS[name](*ins)
        got = got if isinstance(got, tuple) else (got,)
        assert len(got) == len(outs), key
        for g, want in zip(got, outs):
            if want.dtype == torch.int8:
                assert torch.equal(g, want), key
            else:
                # same formulas in the same precision: agreement to rounding noise, far
                # inside the reference's own tolerance (atol = rtol = 2e-2 .. 1e-6)
                torch.testing.assert_close(g, want, rtol=2e-6, atol=2e-7)
        seen += 1
    assert seen >= 2


def test_golden_file_has_all_six_reference_workloads(golden):
    names = {k.split("/")[0] for k in golden.files}
    assert names == set(O.REFERENCE_FUNCTIONS)


def test_layernorm_backward_stats_dx_agrees_with_reference_formula():
    """With statistics computed from x, the given-statistics form reduces to the pinned one."""
    torch.manual_seed(3)
    x = torch.rand(6, 500) * 2 - 1
    dy = torch.rand(6, 500) * 2 - 1
    gamma = torch.rand(500) * 0.5 + 0.75
    mean = x.mean(dim=-1)
    rstd = torch.rsqrt((x - mean[:, None]).square().mean(dim=-1) + 1e-5)
    dx, dgamma, dbeta = O.layernorm_backward_stats(x, dy, gamma, mean, rstd)
    torch.testing.assert_close(dx, O.layernorm_backward(x, dy, gamma), rtol=1e-5, atol=1e-6)
    xhat = (x - mean[:, None]) * rstd[:, None]
    torch.testing.assert_close(dgamma, (dy * xhat).sum(0))
    torch.testing.assert_close(dbeta, dy.sum(0))


def test_layernorm_backward_stats_matches_autograd():
    torch.manual_seed(4)
    x = torch.randn(5, 320, dtype=torch.float64, requires_grad=True)
    gamma = (torch.rand(320, dtype=torch.float64) + 0.5).requires_grad_()
    beta = torch.zeros(320, dtype=torch.float64, requires_grad=True)
    dy = torch.randn(5, 320, dtype=torch.float64)
    y = torch.nn.functional.layer_norm(x, (320,), gamma, beta, 1e-5)
    y.backward(dy)
    mean = x.detach().mean(-1)
    rstd = torch.rsqrt(x.detach().var(-1, unbiased=False) + 1e-5)
    dx, dgamma, dbeta = O.layernorm_backward_stats(x.detach(), dy, gamma.detach(), mean, rstd,
                                                   dtype=torch.float64)
    torch.testing.assert_close(dx, x.grad, rtol=1e-9, atol=1e-11)
    torch.testing.assert_close(dgamma, gamma.grad, rtol=1e-9, atol=1e-11)
    torch.testing.assert_close(dbeta, beta.grad, rtol=1e-9, atol=1e-11)


def test_layernorm_forward_matches_torch_layer_norm():
    torch.manual_seed(5)
    x = (0.5 + 2.0 * torch.randn(4, 777)).bfloat16()
    gamma = torch.rand(777) + 0.5
    beta = 0.1 * torch.randn(777)
    y, mean, rstd = O.layernorm_forward(x, gamma, beta)
    want = torch.nn.functional.layer_norm(x.float(), (777,), gamma, beta, 1e-5)
    torch.testing.assert_close(y.float(), want.bfloat16().float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(mean, x.float().mean(-1))
    assert y.dtype == torch.bfloat16 and mean.dtype == torch.float32


def test_rmsnorm_forward_fp32_vs_fp64():
    torch.manual_seed(6)
    x = torch.randn(3, 1024)
    gamma = torch.rand(1024) + 0.5
    y32 = O.rmsnorm_forward(x, gamma)
    y64 = O.rmsnorm_forward(x, gamma, dtype=torch.float64)
    torch.testing.assert_close(y32.double(), y64, rtol=1e-5, atol=1e-6)
    want = torch.nn.functional.rms_norm(x, (1024,), gamma, 1e-6)
    torch.testing.assert_close(y32, want, rtol=1e-5, atol=1e-6)


def test_row_reduce_first_maximum_and_planted_value():
    x = torch.tensor([[1.0, 7.0, 7.0, -2.0], [-3.0, -3.0, -5.0, -3.0]])
    s, m, a = O.row_reduce(x)
    assert a.tolist() == [1, 0] and a.dtype == torch.int64
    assert m.tolist() == [7.0, -3.0]
    assert s.tolist() == [13.0, -14.0]


def test_ffn_forward_shapes_and_residual_rmsnorm():
    torch.manual_seed(7)
    x = torch.randn(8, 64).bfloat16()
    w1 = (0.02 * torch.randn(64, 256)).bfloat16()
    w2 = (0.02 * torch.randn(256, 64)).bfloat16()
    gamma = torch.rand(64) + 0.5
    y = O.ffn_forward(x, w1, w2, gamma)
    assert y.shape == (8, 64) and y.dtype == torch.bfloat16
    y64 = O.ffn_forward(x, w1, w2, gamma, dtype=torch.float64, round_hidden=False)
    # RMSNorm output: mean square of y/gamma is 1
    ms = (y64 / gamma.double()).square().mean(-1)
    torch.testing.assert_close(ms, torch.ones_like(ms), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(y.double(), y64, rtol=2e-2, atol=2e-2)


def test_lcg_inputs_follow_the_reference_hash():
    x, dy, gamma = O.lcg_layernorm_inputs(2, 8)
    # element 0: a = 12345 >> 16 = 0 -> x = -1; b = 1013904223 >> 16 = 15470, & 2047 = 1134
    assert x[0, 0].item() == -1.0
    assert dy[0, 0].item() == pytest.approx(1134 / 1024.0 - 1.0)
    a1 = ((1103515245 + 12345) >> 16) & 0xFFFFFFFF
    assert x[0, 1].item() == pytest.approx((a1 & 2047) / 1024.0 - 1.0)
    assert gamma[3].item() == pytest.approx(0.75 + 3 * 0.015625)
    q = O.lcg_quant_input(1, 4)
    assert q.shape == (1, 4) and q.dtype == torch.float32
