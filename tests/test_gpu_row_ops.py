"""Parity of the five reference-sweep workloads (weighted variance, Pearson, softmax
backward, LARS, int8 quantisation) through the C ABI:

* against the reference's OWN outputs on the stored golden inputs
  (tests/golden/reference_workloads.npz, made by importing the reference);
* against the CPU oracle (the pinned restatement, evaluated in fp64) on seeded
  inputs of the reference's distributions, for every cluster size, ragged and
  unaligned widths, and the no-staging variant.

Tolerances are the reference's own (dsmem_eval/workloads.py:164-210): atol = rtol =
3e-2 (weighted variance), 3e-3 (Pearson, softmax, LARS), 1e-6 for the quantiser's
scale; int8 values may differ by one at a rate of at most 1e-5 (runner.py:198-215),
and are bit-exact on the golden inputs.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

from credit_b200 import _native as N
from credit_b200 import launchers as L
from credit_b200 import workloads as W
from oracle import reference_ops as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_workloads.npz"
ROW_OPS = ["weighted_var_backward", "pearson_backward", "softmax_logits_backward", "lars_momentum",
           "rowwise_quant"]
WORKLOAD_IDS = {"weighted_var_backward": N.WL_WEIGHTED_VAR_BACKWARD, "pearson_backward": N.WL_PEARSON_BACKWARD,
                "softmax_logits_backward": N.WL_SOFTMAX_LOGITS_BACKWARD, "lars_momentum": N.WL_LARS_MOMENTUM,
                "rowwise_quant": N.WL_ROWWISE_QUANT}


def run(name, inputs, cluster_size=0, opts=None):
    ins = tuple(t.to(DEV).contiguous() for t in inputs)
    outs = L.allocate_outputs(name, ins)
    for o in outs:
        o.fill_(99 if o.dtype == torch.int8 else float("nan"))
    L.NATIVE_LAUNCHERS[name](ins, outs, cluster_size, opts)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    return tuple(o.cpu() for o in outs)


def compare(name, got, want, exact_int8=False):
    spec = W.WORKLOADS[name]
    assert len(got) == len(want)
    for g, w in zip(got, want):
        if g.dtype == torch.int8:
            diff = (g.to(torch.int16) - w.to(torch.int16)).abs()
            if exact_int8:
                assert int(diff.max()) == 0
            else:
                assert int(diff.max()) <= 1 and float((diff != 0).float().mean()) <= 1.0e-5
        else:
            w32 = w.to(torch.float32).reshape(g.shape)
            assert torch.allclose(g, w32, atol=spec.atol, rtol=spec.rtol), \
                f"{name}: max error {float((g - w32).abs().max()):.3e}"


def oracle64(name, inputs):
    out = O.REFERENCE_FUNCTIONS[name](*(t.double() for t in inputs))
    out = out if isinstance(out, tuple) else (out,)
    if name == "rowwise_quant":      # quantise in fp32 as the reference does: rounding ties depend on it
        out = O.REFERENCE_FUNCTIONS[name](*inputs)
    return out


@pytest.mark.parametrize("name", ROW_OPS)
@pytest.mark.parametrize("cluster_size", [0, 1, 2, 4, 8, 16])
def test_golden_inputs_reproduce_reference_outputs(native_lib, name, cluster_size):
    golden = np.load(GOLDEN)
    for shape in ("3x96", "2x1000"):
        ins, outs = [], []
        i = 0
        while f"{name}/{shape}/in{i}" in golden.files:
            ins.append(torch.from_numpy(golden[f"{name}/{shape}/in{i}"]))
            i += 1
        i = 0
        while f"{name}/{shape}/out{i}" in golden.files:
            outs.append(torch.from_numpy(golden[f"{name}/{shape}/out{i}"]))
            i += 1
        compare(name, run(name, ins, cluster_size), outs, exact_int8=True)


@pytest.mark.parametrize("name", ROW_OPS)
@pytest.mark.parametrize("rows,cols,cluster_size", [
    (64, 4096, 0), (64, 4096, 2), (33, 16384, 4), (17, 32768, 8), (9, 65536, 16), (5, 65536, 8),
    (7, 1000, 4), (3, 97, 16), (4, 33333, 8), (6, 4099, 2), (2, 1, 2), (300, 8192, 8),
])
def test_matches_oracle(native_lib, name, rows, cols, cluster_size):
    inputs = W.WORKLOADS[name].input_factory(rows, cols, "cpu", seed=rows + cols)
    compare(name, run(name, inputs, cluster_size), oracle64(name, inputs))


@pytest.mark.parametrize("name", ROW_OPS)
@pytest.mark.parametrize("threads", [256, 512])
@pytest.mark.parametrize("rows,cols,cluster_size", [(64, 4096, 0), (33, 16384, 4), (9, 65536, 16), (300, 8192, 8)])
def test_lock_step_kernels(native_lib, name, threads, rows, cols, cluster_size):
    """threads = 256 / 512 keep the staged kernels that make one pass and one cluster barrier per
    dependent reduction (the automatic choice for aligned rows is the warp-specialised pipeline)."""
    inputs = W.WORKLOADS[name].input_factory(rows, cols, "cpu", seed=rows + cols)
    opts = {"threads": threads}
    compare(name, run(name, inputs, cluster_size, opts), oracle64(name, inputs))
    assert N.plan(WORKLOAD_IDS[name], rows, cols, N.F32, dict(opts, cluster_size=cluster_size)).threads == threads


@pytest.mark.parametrize("name", ROW_OPS)
@pytest.mark.parametrize("cluster_size,stages", [(1, 0), (2, 3), (4, 4), (8, 0), (16, 5)])
def test_warp_specialised_pipeline_many_rows(native_lib, name, cluster_size, stages):
    """threads = 352 on aligned rows: 20+ rows per cluster, so the ring and every buffer of the
    pipeline wrap; the second shape leaves CTAs with short and empty slices."""
    opts = {"threads": 352, "stages": stages}
    for rows, cols in ((3100, 2048), (2999, 1096)):
        inputs = W.WORKLOADS[name].input_factory(rows, cols, "cpu", seed=rows)
        compare(name, run(name, inputs, cluster_size, opts), oracle64(name, inputs))
        assert N.plan(WORKLOAD_IDS[name], rows, cols, N.F32, dict(opts, cluster_size=cluster_size)).threads == 352


def test_softmax_extreme_logits(native_lib):
    """Online softmax: a row whose maximum arrives late, rows of equal logits, -inf entries and a
    huge dynamic range give the same result as the three-pass formula."""
    rows, cols = 6, 8192
    torch.manual_seed(2)
    logits = torch.randn(rows, cols) * 3.0
    logits[0, cols - 1] = 80.0                    # the maximum is the last element
    logits[1, :] = 1.5                            # all equal
    logits[2, 100:200] = float("-inf")            # masked entries
    logits[3, :] = torch.linspace(-200.0, 50.0, cols)
    logits[4, 0] = 60.0                           # the maximum is the first element
    dy = torch.randn(rows, cols)
    want = O.softmax_logits_backward(logits.double(), dy.double()).float()
    for p in (1, 4, 16):
        (got,) = run("softmax_logits_backward", (logits, dy), p)
        assert torch.allclose(got, want, atol=3e-6, rtol=3e-3), float((got - want).abs().max())


@pytest.mark.parametrize("name", ["pearson_backward", "weighted_var_backward"])
def test_shifted_moments_with_a_large_offset(native_lib, name):
    """mean >> spread: the one-pass shifted moments keep the centred sums accurate."""
    rows, cols = 5, 16384
    inputs = list(W.WORKLOADS[name].input_factory(rows, cols, "cpu", seed=4))
    inputs[0] = inputs[0] * 0.01 + 300.0
    if name == "pearson_backward":
        inputs[1] = inputs[1] * 0.01 - 120.0
    want = oracle64(name, inputs)
    got = run(name, inputs, 8)
    for g, w in zip(got, want):
        w = w.float()
        assert torch.allclose(g, w, atol=3e-3 * float(w.abs().max()), rtol=3e-3), float((g - w).abs().max())


@pytest.mark.parametrize("name", ROW_OPS)
@pytest.mark.parametrize("cols", [4096, 4099, 65536])
def test_no_staging_variant(native_lib, name, cols):
    inputs = W.WORKLOADS[name].input_factory(12, cols, "cpu", seed=cols)
    got = run(name, inputs, 0, {"variant": N.VARIANT_BLOCK_READ})
    compare(name, got, oracle64(name, inputs))


@pytest.mark.parametrize("name", ROW_OPS)
def test_unaligned_base_pointer(native_lib, name):
    rows, cols = 5, 2048
    inputs = W.WORKLOADS[name].input_factory(rows, cols, "cpu", seed=11)
    ins = []
    for t in inputs:
        if t.shape == (rows, cols):       # shift the matrix by one element inside a larger buffer
            buf = torch.empty(rows * cols + 1, device=DEV)
            view = buf[1:].view(rows, cols)
            view.copy_(t)
            ins.append(view)
        else:
            ins.append(t.to(DEV))
    outs = L.allocate_outputs(name, tuple(ins))
    L.NATIVE_LAUNCHERS[name](tuple(ins), outs, 4)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    compare(name, tuple(o.cpu() for o in outs), oracle64(name, inputs))


def test_quantiser_edge_rows(native_lib):
    x = torch.zeros(4, 512)
    x[1, 7] = -3.0                      # single non-zero element: q = -127 there
    x[2] = torch.linspace(-1, 1, 512)
    x[3] = 0.5                          # every element at the maximum
    q, scale = run("rowwise_quant", (x,), 2)
    want_q, want_scale = O.rowwise_quant(x)
    assert torch.equal(q, want_q)
    assert torch.allclose(scale, want_scale, rtol=1e-6, atol=0)
    assert int(q[0].abs().max()) == 0 and float(scale[0]) == 0.0


def test_row_op_argument_errors(native_lib):
    x = torch.zeros(4, 256, device=DEV)
    lib = N.load()
    # missing second input of a two-input workload
    rc = lib.credit_row_op(N.WL_SOFTMAX_LOGITS_BACKWARD, x.data_ptr(), None, None, None, x.data_ptr(), None, None,
                           4, 256, None, None)
    assert rc == N.ERR_INVALID_ARGUMENT
    # a workload id of another family
    rc = lib.credit_row_op(N.WL_RMSNORM_FORWARD, x.data_ptr(), None, None, None, x.data_ptr(), None, None, 4, 256,
                           None, None)
    assert rc == N.ERR_INVALID_ARGUMENT
    # empty batch is a no-op
    e = torch.zeros(0, 256, device=DEV)
    L.NATIVE_LAUNCHERS["rowwise_quant"]((e,), L.allocate_outputs("rowwise_quant", (e,)))


@pytest.mark.parametrize("name", ROW_OPS)
def test_512_thread_kernels(native_lib, name):
    inputs = W.WORKLOADS[name].input_factory(10, 16384, "cpu", seed=21)
    compare(name, run(name, inputs, 4, {"threads": 512}), oracle64(name, inputs))
    compare(name, run(name, inputs, 0, {"threads": 512, "variant": N.VARIANT_BLOCK_READ}), oracle64(name, inputs))
