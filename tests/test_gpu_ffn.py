"""Parity of the tcgen05 FFN against the CPU oracle, through the C ABI.
Tolerance: bf16 outputs, 2e-2 relative (+ 2e-2 absolute on O(1) normalised outputs)."""
import pytest
import torch

from credit_b200 import _native as N
from credit_b200 import launchers as L
from credit_b200 import workloads as W
from oracle import reference_ops as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def run_ffn(x, w1, w2, gamma):
    xd, w1d, w2d, gd = (t.to(DEV) for t in (x, w1, w2, gamma))
    w1p, w2p = L.pack_ffn_weight(w1d), L.pack_ffn_weight(w2d)
    y = torch.full_like(xd, float("nan"))
    L.launch_ffn_forward((xd, w1p, w2p, gd), (y,))
    torch.cuda.synchronize()
    assert N.device_status() == 0
    return y.cpu(), w1p.cpu()


def check(y, want):
    err = (y.double() - want.double()).abs()
    bound = 2e-2 * want.double().abs() + 2e-2
    assert bool((err <= bound).all()), f"worst error {float(err.max()):.3e}"


@pytest.mark.parametrize("m,d,h", [(128, 256, 512), (256, 512, 1024), (128, 1024, 2048), (384, 2048, 512),
                                    (128, 4096, 1024), (1024, 512, 8192),
                                    # more row blocks than resident clusters: the second GEMM splits blocks by k range
                                    (1152, 4096, 512), (2048, 2048, 768),
                                    # two row blocks at a time per cluster (both accumulators, one B tile): one round
                                    # of pairs plus a split tail; two rounds of pairs; pairs, a single round and a tail
                                    (2048, 4096, 512), (3584, 4096, 256), (3072, 4096, 256)])
def test_ffn_forward_matches_oracle(native_lib, m, d, h):
    x, w1, w2, gamma = W.make_ffn_inputs(m, d, "cpu", seed=m + d, hidden=h)
    y, w1p = run_ffn(x, w1, w2, gamma)
    assert torch.equal(w1p, w1.t().contiguous()), "packing is a transposition"
    check(y, O.ffn_forward(x, w1, w2, gamma, dtype=torch.float64))


def test_ffn_forward_headline_shape_row_sample(native_lib):
    """Full shape on the GPU; the oracle checks a sample of rows (rows are independent)."""
    m, d, h = 2048, 4096, 16384
    x, w1, w2, gamma = W.make_ffn_inputs(m, d, "cpu", seed=0, hidden=h)
    y, _ = run_ffn(x, w1, w2, gamma)
    # rows of every row block (blocks 2, 4, 6, 9, 11 and 13 are split between two clusters when 7 are resident)
    rows = torch.tensor([0, 1, 127, 128, 300, 383, 600, 777, 900, 1000, 1200, 1290, 1500, 1700, 1800, 2047])
    want = O.ffn_forward(x[rows], w1, w2, gamma, dtype=torch.float32)
    check(y[rows], want)
    # RMSNorm property over the whole output: mean square of y / gamma is 1 for every row
    ms = (y.float() / gamma).square().mean(-1)
    assert bool(((ms - 1.0).abs() < 2e-2).all())


def test_ffn_rejects_unsupported_shapes(native_lib):
    x, w1, w2, gamma = (t.to(DEV) for t in W.make_ffn_inputs(100, 256, "cpu", hidden=512))
    with pytest.raises(N.UnsupportedShape):
        L.launch_ffn_forward((x, L.pack_ffn_weight(w1), L.pack_ffn_weight(w2), gamma), (torch.empty_like(x),))
    assert N.load().credit_ffn_workspace_bytes(128, 8192, 512) == 0      # d above 4096
