"""Parity of the CUDA path against the CPU oracle, through the C ABI
(ctypes -> libcredit_b200.so), on seeded inputs the oracle finishes in seconds.

Tolerances: fp32 outputs 1e-5 relative, bf16 outputs 2e-2 relative, argmax exact.
"Relative" is applied as |got - want| <= rtol * |want| + atol with an atol equal to
rtol times the natural scale of the quantity, because rows whose true value is near
zero make a purely relative test ill-posed (the reference does the same with its
atol + rtol * |ref| checks, dsmem_eval/runner.py:218).
"""
import pytest
import torch

from credit_b200 import _native as N
from credit_b200 import launchers as L
from credit_b200 import workloads as W
from oracle import reference_ops as O

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")
CLUSTER_SIZES = [1, 2, 4, 8, 16]
FP32_RTOL = 1.0e-5
BF16_RTOL = 2.0e-2

# (rows, cols): aligned rows, rows narrower than the cluster, ragged widths, one-element rows
ALIGNED_SHAPES = [(1, 256), (7, 4096), (40, 8192), (3, 64), (300, 1024)]
RAGGED_SHAPES = [(3, 1000), (4, 97), (2, 33333), (5, 1), (2, 4099)]


@pytest.fixture(autouse=True)
def _healthy_device(native_lib):
    yield
    assert N.device_status() == 0, "a kernel reported a timeout or bad geometry"


def to_dev(tensors):
    return tuple(t.to(DEV) for t in tensors)


def run(name, inputs, cluster_size=0, opts=None, **kw):
    dev_inputs = to_dev(inputs)
    outputs = L.allocate_outputs(name, dev_inputs)
    for o in outputs:
        if o.dtype.is_floating_point:
            o.fill_(float("nan"))
        else:
            o.fill_(-7)
    L.NATIVE_LAUNCHERS[name](dev_inputs, outputs, cluster_size, opts, **kw)
    torch.cuda.synchronize()
    return tuple(o.cpu() for o in outputs)


def try_run(name, inputs, cluster_size, opts=None, **kw):
    """Runs, or skips when the shape does not fit the variant (the reference prints n/a)."""
    try:
        return run(name, inputs, cluster_size, opts, **kw)
    except N.UnsupportedShape as exc:
        pytest.skip(str(exc))


def close(got, want, rtol, scale=1.0, what=""):
    got = got.double()
    want = want.double()
    err = (got - want).abs()
    bound = rtol * want.abs() + rtol * scale
    bad = err > bound
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())} of {bad.numel()} outside tolerance; worst error "
        f"{float(err.max()):.3e} at value {float(want.flatten()[err.argmax()]):.3e}")


# ---------------------------------------------------------------------------
# RMSNorm forward
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("cluster_size", CLUSTER_SIZES)
@pytest.mark.parametrize("shape", ALIGNED_SHAPES + RAGGED_SHAPES)
def test_rmsnorm_forward_fp32(shape, cluster_size):
    rows, cols = shape
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=rows + cols)
    (y,) = try_run("rmsnorm_forward", (x, gamma), cluster_size)
    want = O.rmsnorm_forward(x, gamma, dtype=torch.float64)
    close(y, want, FP32_RTOL, scale=1.0, what="y")


@pytest.mark.parametrize("cluster_size", [1, 4, 16])
@pytest.mark.parametrize("shape", [(5, 4096), (3, 1000), (2, 264)])
def test_rmsnorm_forward_bf16(shape, cluster_size):
    rows, cols = shape
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=1)
    x = x.bfloat16()
    (y,) = try_run("rmsnorm_forward", (x, gamma), cluster_size)
    want = O.rmsnorm_forward(x, gamma, dtype=torch.float64)
    close(y, want, BF16_RTOL, scale=1.0, what="y")


@pytest.mark.parametrize("opts", [
    {"schedule": N.SCHEDULE_ROW_PER_CLUSTER},
    {"schedule": N.SCHEDULE_PERSISTENT, "stages": 1},
    {"schedule": N.SCHEDULE_PERSISTENT, "stages": 3},
    {"schedule": N.SCHEDULE_PERSISTENT, "stages": 4, "threads": 512},
    {"variant": N.VARIANT_BLOCK_SMEM},
    {"variant": N.VARIANT_CLUSTER_SMEM},
])
def test_rmsnorm_forward_schedules_and_rings(opts):
    """More rows than resident clusters, so persistent clusters walk several rows and the
    ring wraps."""
    rows, cols = 2500, 2048
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=11)
    (y,) = try_run("rmsnorm_forward", (x, gamma), opts.get("cluster_size", 0), opts)
    close(y, O.rmsnorm_forward(x, gamma, dtype=torch.float64), FP32_RTOL, what="y")


def test_rmsnorm_forward_headline_width():
    rows, cols = 64, 32768
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=0)
    for p in (1, 2, 4, 8, 16):
        (y,) = run("rmsnorm_forward", (x, gamma), p)
        close(y, O.rmsnorm_forward(x, gamma, dtype=torch.float64), FP32_RTOL, what=f"y P={p}")


def test_rmsnorm_unaligned_base_pointer_takes_the_scalar_path():
    rows, cols = 6, 1024
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=2)
    big = torch.empty(rows * cols + 1, device=DEV, dtype=torch.float32)
    xd = big[1:].view(rows, cols)          # 4-byte aligned only
    xd.copy_(x)
    y = torch.empty(rows, cols, device=DEV)
    L.launch_rmsnorm_forward((xd, gamma.to(DEV)), (y,), 2)
    torch.cuda.synchronize()
    close(y.cpu(), O.rmsnorm_forward(x, gamma, dtype=torch.float64), FP32_RTOL, what="y")


# ---------------------------------------------------------------------------
# Row reduction: sum, max, argmax
# ---------------------------------------------------------------------------
def check_row_reduce(x, got):
    s, m, a = got
    want_s, want_m, want_a = O.row_reduce(x, dtype=torch.float64)
    assert a.dtype == torch.int64
    assert torch.equal(a, want_a), "argmax must be bit-exact"
    assert torch.equal(m, want_m), "max must be bit-exact"
    # natural scale of a sum of `cols` O(1) terms
    close(s, want_s, FP32_RTOL, scale=float(x.abs().sum(-1).max()) / max(1.0, x.shape[1] ** 0.5), what="sum")


@pytest.mark.parametrize("load_path", [N.LOAD_TMA, N.LOAD_LDG])
@pytest.mark.parametrize("cluster_size", CLUSTER_SIZES)
@pytest.mark.parametrize("shape", [(3, 4096), (17, 65536), (2, 262144 + 64), (9, 256)])
def test_row_reduce_aligned(shape, cluster_size, load_path):
    rows, cols = shape
    (x,) = W.make_row_reduce_inputs(rows, cols, "cpu", seed=rows)
    got = try_run("row_reduce", (x,), cluster_size, {"load_path": load_path})
    check_row_reduce(x, got)


@pytest.mark.parametrize("cluster_size", [1, 2, 8, 16])
@pytest.mark.parametrize("shape", RAGGED_SHAPES)
def test_row_reduce_ragged(shape, cluster_size):
    rows, cols = shape
    (x,) = W.make_row_reduce_inputs(rows, cols, "cpu", seed=cols)
    check_row_reduce(x, try_run("row_reduce", (x,), cluster_size))


@pytest.mark.parametrize("opts", [
    {"load_path": N.LOAD_TMA, "stages": 2, "chunk_bytes": 4096},
    {"load_path": N.LOAD_TMA, "stages": 8, "chunk_bytes": 1024},
    {"load_path": N.LOAD_TMA, "stages": 3, "chunk_bytes": 32768, "threads": 512},
    {"load_path": N.LOAD_TMA, "schedule": N.SCHEDULE_ROW_PER_CLUSTER},
    {"load_path": N.LOAD_LDG, "schedule": N.SCHEDULE_PERSISTENT},
    {"load_path": N.LOAD_LDG, "threads": 512},
])
@pytest.mark.parametrize("cluster_size", [1, 4])
def test_row_reduce_rings_and_schedules(opts, cluster_size):
    rows, cols = 1500, 10240
    (x,) = W.make_row_reduce_inputs(rows, cols, "cpu", seed=5)
    check_row_reduce(x, try_run("row_reduce", (x,), cluster_size, opts))


@pytest.mark.parametrize("load_path", [N.LOAD_TMA, N.LOAD_LDG])
def test_row_reduce_ties_take_the_lowest_column(load_path):
    rows, cols = 4, 8192
    x = torch.zeros(rows, cols)
    x[0, [5000, 17, 8000]] = 3.0          # tie across CTAs and threads
    x[1, :] = -1.0                        # every element equal
    x[2, cols - 1] = 1.0                  # last column
    x[3, :] = float("-inf")               # nothing beats the initial value
    for p in (1, 2, 8):
        s, m, a = run("row_reduce", (x,), p, {"load_path": load_path})
        assert a.tolist() == [17, 0, cols - 1, 0], (p, a.tolist())
        assert m[:3].tolist() == [3.0, -1.0, 1.0]
        assert m[3].item() == float("-inf")


@pytest.mark.parametrize("load_path", [N.LOAD_TMA, N.LOAD_LDG])
@pytest.mark.parametrize("cols", [65536, 33333])
def test_row_reduce_nan_propagates_like_torch(load_path, cols):
    """torch.amax / torch.argmax (the oracle) let a NaN win over every number and report the FIRST
    NaN's column; the row sum is NaN. +inf and -inf in one row make the sum NaN without any NaN
    element: maximum and argmax then stay ordinary."""
    if load_path == N.LOAD_TMA and cols % 4:
        pytest.skip("bulk copies need 16-byte rows")
    rows = 6
    torch.manual_seed(3)
    x = torch.randn(rows, cols)
    nan, inf = float("nan"), float("inf")
    x[0, cols - 1] = nan                                   # last column, last CTA
    x[1, [40000 % cols, 123, 30000]] = nan                 # several: the lowest column counts
    x[1, 7] = inf                                          # an infinity before the first NaN loses to it
    x[2, 0] = nan                                          # first column
    x[3, 100] = inf
    x[3, 20000] = -inf                                     # sum is NaN, no NaN element
    x[4, :] = nan                                          # every element
    want_sum, want_max, want_arg = O.row_reduce(x)
    assert want_arg.tolist()[:5] == [cols - 1, 123, 0, 100, 0]
    for p in (1, 4, 16):
        s, m, a = run("row_reduce", (x,), p, {"load_path": load_path})
        assert torch.equal(a, want_arg), (p, a.tolist())
        assert torch.equal(torch.isnan(m), torch.isnan(want_max))
        assert torch.equal(m[~torch.isnan(m)], want_max[~torch.isnan(want_max)])
        assert torch.equal(torch.isnan(s), torch.isnan(want_sum))
        assert bool(torch.isnan(s[:5]).all()) and not bool(torch.isnan(s[5]))


def test_row_reduce_headline_width_few_rows():
    rows, cols = 6, 1048576
    (x,) = W.make_row_reduce_inputs(rows, cols, "cpu", seed=0)
    for p in (4, 8, 16):
        for path in (N.LOAD_TMA, N.LOAD_LDG):
            check_row_reduce(x, run("row_reduce", (x,), p, {"load_path": path}))


# ---------------------------------------------------------------------------
# LayerNorm forward
# ---------------------------------------------------------------------------
def check_layernorm_forward(inputs, got, rtol_y):
    x, gamma, beta = inputs
    y, mean, rstd = got
    want_y, want_mean, want_rstd = O.layernorm_forward(x, gamma, beta, dtype=torch.float64)
    # statistics are fp32 outputs whatever the storage type of x
    spread = float(x.double().std()) if x.numel() > 1 else 1.0
    close(mean, want_mean, FP32_RTOL, scale=max(spread, 1e-3), what="mean")
    close(rstd, want_rstd, FP32_RTOL, what="rstd")
    close(y, want_y, rtol_y, scale=1.0, what="y")


@pytest.mark.parametrize("cluster_size", CLUSTER_SIZES)
@pytest.mark.parametrize("shape", ALIGNED_SHAPES + RAGGED_SHAPES)
def test_layernorm_forward_bf16(shape, cluster_size):
    rows, cols = shape
    inputs = W.make_layernorm_forward_inputs(rows, cols, "cpu", seed=rows * 3 + cols)
    check_layernorm_forward(inputs, try_run("layernorm_forward", inputs, cluster_size), BF16_RTOL)


@pytest.mark.parametrize("cluster_size", [1, 2, 8])
@pytest.mark.parametrize("shape", [(9, 4096), (3, 1000), (2, 12)])
def test_layernorm_forward_fp32(shape, cluster_size):
    rows, cols = shape
    inputs = W.make_layernorm_forward_inputs(rows, cols, "cpu", seed=9, dtype=torch.float32)
    check_layernorm_forward(inputs, try_run("layernorm_forward", inputs, cluster_size), FP32_RTOL)


def test_layernorm_forward_large_offset_has_no_cancellation():
    """mean >> std: the slice-centred statistics keep the variance accurate."""
    rows, cols = 4, 8192
    torch.manual_seed(0)
    x = 1000.0 + 0.01 * torch.randn(rows, cols)
    gamma = torch.ones(cols)
    beta = torch.zeros(cols)
    for p in (1, 4, 16):
        y, mean, rstd = run("layernorm_forward", (x, gamma, beta), p)
        _, want_mean, want_rstd = O.layernorm_forward(x, gamma, beta, dtype=torch.float64)
        close(mean, want_mean, FP32_RTOL, scale=0.0, what="mean")
        close(rstd, want_rstd, 1.0e-3, what="rstd")   # limited by fp32 storage of x itself


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sigmas", [100.0, 1000.0])
def test_layernorm_statistics_survive_an_outlier_in_the_first_column(dtype, sigmas):
    """x[:, 0] far from the row mean: a one-pass variance shifted by the row's first element
    would lose 1e-3 and more of the variance to cancellation. Covers the forward and the
    statistics-recomputing backward on the register path (aligned rows) at several cluster sizes."""
    rows, cols = 6, 65536
    torch.manual_seed(11)
    x = torch.randn(rows, cols)
    x[:, 0] = sigmas
    x[1, cols - 1] = -sigmas          # one row with two outliers, one of them a sampled position
    x = x.to(dtype)
    gamma = torch.rand(cols) + 0.5
    beta = torch.zeros(cols)
    dy = torch.randn(rows, cols).to(dtype)
    _, want_mean, want_rstd = O.layernorm_forward(x, gamma, beta, dtype=torch.float64)
    want_dx = O.layernorm_backward(x.double(), dy.double(), gamma.double())
    for p, opts in ((2, None), (8, None), (16, None), (8, {"threads": 608}), (16, {"threads": 352}), (8, {"threads": 512})):
        y, mean, rstd = run("layernorm_forward", (x, gamma, beta), p, opts)
        close(rstd, want_rstd, FP32_RTOL, what=f"rstd P={p}")
        close(mean, want_mean, FP32_RTOL, scale=1.0, what=f"mean P={p}")
    for p in (4, 8, 16):   # x and dy staged: two fp32 half rows do not fit one CTA
        (dx,) = run("layernorm_backward", (x, dy, gamma), p)
        close(dx, want_dx, FP32_RTOL if dtype == torch.float32 else BF16_RTOL, scale=2.0, what=f"dx P={p}")


def test_layernorm_forward_headline_width():
    rows, cols = 24, 131072
    inputs = W.make_layernorm_forward_inputs(rows, cols, "cpu", seed=0)
    for p in (2, 4, 8, 16):
        check_layernorm_forward(inputs, run("layernorm_forward", inputs, p), BF16_RTOL)


@pytest.mark.parametrize("opts", [
    {"schedule": N.SCHEDULE_ROW_PER_CLUSTER},
    {"schedule": N.SCHEDULE_PERSISTENT, "stages": 2},
    {"schedule": N.SCHEDULE_PERSISTENT, "stages": 4, "threads": 512},
])
def test_layernorm_forward_many_rows(opts):
    rows, cols = 3000, 1536
    inputs = W.make_layernorm_forward_inputs(rows, cols, "cpu", seed=4)
    check_layernorm_forward(inputs, try_run("layernorm_forward", inputs, 0, opts), BF16_RTOL)


# ---------------------------------------------------------------------------
# LayerNorm backward, reference form (statistics recomputed, dx only)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("cluster_size", CLUSTER_SIZES)
@pytest.mark.parametrize("shape", ALIGNED_SHAPES + RAGGED_SHAPES)
def test_layernorm_backward_reference_form_fp32(shape, cluster_size):
    rows, cols = shape
    inputs = W.make_layernorm_inputs(rows, cols, "cpu", seed=rows + 7 * cols)
    (dx,) = try_run("layernorm_backward", inputs, cluster_size)
    want = O.layernorm_backward(*[t.double() for t in inputs])
    # dx of a row is O(1 / std(x)) ~ 1.7 for U(-1,1); single-element rows give exactly 0
    close(dx, want, FP32_RTOL, scale=2.0, what="dx")


def test_layernorm_backward_on_the_reference_binary_inputs():
    """Inputs of the reference executable (index hashes), reference tolerance 2e-2
    (layernorm_backward.cu:665) and the tighter fp32 bound."""
    rows, cols = 16, 4096
    inputs = O.lcg_layernorm_inputs(rows, cols)
    want = O.layernorm_backward(*[t.double() for t in inputs])
    for p in (2, 4, 8):
        (dx,) = run("layernorm_backward", inputs, p)
        assert bool(((dx.double() - want).abs() <= 2e-2 + 2e-2 * want.abs()).all())
        close(dx, want, FP32_RTOL, scale=2.0, what="dx")


@pytest.mark.parametrize("cluster_size", [1, 4, 16])
def test_layernorm_backward_reference_form_bf16(cluster_size):
    rows, cols = 12, 8192
    x, dy, gamma = W.make_layernorm_inputs(rows, cols, "cpu", seed=21)
    x, dy = x.bfloat16(), dy.bfloat16()
    (dx,) = try_run("layernorm_backward", (x, dy, gamma), cluster_size)
    want = O.layernorm_backward(x.double(), dy.double(), gamma.double())
    close(dx, want, BF16_RTOL, scale=2.0, what="dx")


# ---------------------------------------------------------------------------
# LayerNorm backward with given statistics: dx, dgamma, dbeta
# ---------------------------------------------------------------------------
def check_backward_stats(inputs, got, rtol_dx):
    x, dy, gamma, mean, rstd = inputs
    dx, dgamma, dbeta = got
    want_dx, want_dg, want_db = O.layernorm_backward_stats(x, dy, gamma, mean, rstd,
                                                           dtype=torch.float64)
    rows = x.shape[0]
    close(dx, want_dx, rtol_dx, scale=2.0, what="dx")
    # column sums of `rows` O(1) terms, accumulated in fp32
    close(dgamma, want_dg, FP32_RTOL, scale=max(1.0, rows ** 0.5) * 4.0, what="dgamma")
    close(dbeta, want_db, FP32_RTOL, scale=max(1.0, rows ** 0.5) * 4.0, what="dbeta")


@pytest.mark.parametrize("cluster_size", CLUSTER_SIZES)
@pytest.mark.parametrize("shape", ALIGNED_SHAPES + RAGGED_SHAPES + [(700, 2048)])
def test_layernorm_backward_stats_bf16(shape, cluster_size):
    rows, cols = shape
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=rows + cols)
    check_backward_stats(inputs, try_run("layernorm_backward_stats", inputs, cluster_size), BF16_RTOL)


@pytest.mark.parametrize("cluster_size", [1, 2, 8])
@pytest.mark.parametrize("shape", [(33, 4096), (3, 1000), (600, 512)])
def test_layernorm_backward_stats_fp32(shape, cluster_size):
    rows, cols = shape
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=3, dtype=torch.float32)
    check_backward_stats(inputs, try_run("layernorm_backward_stats", inputs, cluster_size), FP32_RTOL)


@pytest.mark.parametrize("opts", [
    {"threads": 256, "stages": 2},
    {"threads": 512, "stages": 3},
    {"threads": 512, "stages": 1},
    {"threads": 256, "stages": 4},
])
@pytest.mark.parametrize("cluster_size", [2, 4, 8, 16])
def test_layernorm_backward_stats_register_paths(opts, cluster_size):
    """Every (threads, vectors-per-thread) instantiation with several rows per cluster."""
    rows, cols = 1200, 16384
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=13)
    check_backward_stats(inputs, try_run("layernorm_backward_stats", inputs, cluster_size, opts),
                         BF16_RTOL)


@pytest.mark.parametrize("stages", [0, 3, 4, 5, 8, 16])
@pytest.mark.parametrize("cluster_size", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("threads", [608, 352])
def test_layernorm_backward_stats_warp_specialised_kernel(threads, dtype, cluster_size, stages):
    """threads = 608 / 352: producer, collector and receiver warps and 16 / 8 output warps whose two passes
    run one or two rows apart (by ring depth). 20+ rows per cluster, so the ring, the four CTA-local
    partial buffers and the eight cluster slot buffers all wrap several times; the second shape
    leaves ragged tiles and CTAs with empty slices."""
    opts = {"threads": threads, "stages": stages}
    for rows, cols in ((3100, 4096), (2999, 1096)):
        inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=rows, dtype=dtype)
        got = try_run("layernorm_backward_stats", inputs, cluster_size, opts)
        check_backward_stats(inputs, got, BF16_RTOL if dtype == torch.bfloat16 else FP32_RTOL)
        plan = N.plan(N.WL_LAYERNORM_BACKWARD_STATS, rows, cols, N.BF16 if dtype == torch.bfloat16 else N.F32,
                      dict(opts, cluster_size=cluster_size))
        assert plan.threads == threads and plan.stages >= 3


@pytest.mark.parametrize("stages", [0, 3, 5, 13])
@pytest.mark.parametrize("cluster_size", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("threads", [608, 352])
def test_forward_warp_specialised_kernels(threads, dtype, cluster_size, stages):
    """RMSNorm and LayerNorm forward on the warp-specialised pipeline (threads = 608 / 352): many
    rows per cluster so every ring and buffer wraps; an aligned-but-ragged width leaves partial
    tiles and empty slices; a wide row exercises the largest vector counts."""
    opts = {"threads": threads, "stages": stages}
    for rows, cols in ((2500, 2048), (1999, 1096), (40, 16384 * cluster_size if cluster_size <= 4 else 65536)):
        x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=rows)
        x = x.to(dtype)
        (y,) = try_run("rmsnorm_forward", (x, gamma), cluster_size, opts)
        close(y, O.rmsnorm_forward(x, gamma, dtype=torch.float64), BF16_RTOL if dtype == torch.bfloat16 else FP32_RTOL,
              what="rmsnorm y")
        inputs = W.make_layernorm_forward_inputs(rows, cols, "cpu", seed=rows + 1, dtype=dtype)
        got = try_run("layernorm_forward", inputs, cluster_size, opts)
        check_layernorm_forward(inputs, got, BF16_RTOL if dtype == torch.bfloat16 else FP32_RTOL)
        code = N.BF16 if dtype == torch.bfloat16 else N.F32
        assert N.plan(N.WL_LAYERNORM_FORWARD, rows, cols, code, dict(opts, cluster_size=cluster_size)).threads == threads


@pytest.mark.parametrize("stages", [0, 3, 5])
@pytest.mark.parametrize("cluster_size", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_layernorm_backward_reference_form_warp_specialised_kernel(dtype, cluster_size, stages):
    """The reference form (statistics recomputed from the row, layernorm_backward.cu:217-251 does it
    with two exchanges) as one pass with a record of four shifted sums: many rows per cluster so the
    buffers wrap, a ragged width, a wide row, and rows far from zero (mean 1000, std 0.01) where an
    unshifted sum of squares would cancel."""
    opts = {"threads": 352, "stages": stages}
    rtol = BF16_RTOL if dtype == torch.bfloat16 else FP32_RTOL
    code = N.BF16 if dtype == torch.bfloat16 else N.F32
    for rows, cols in ((3100, 4096), (2999, 1096), (40, 16384 * cluster_size if cluster_size <= 4 else 65536)):
        x, dy, gamma = W.make_layernorm_inputs(rows, cols, "cpu", seed=rows + cols)
        x, dy = x.to(dtype), dy.to(dtype)
        try:
            (dx,) = run("layernorm_backward", (x, dy, gamma), cluster_size, opts)
        except N.UnsupportedShape:
            assert cols > 4096   # only the wide row may exceed a small cluster's shared memory
            continue
        close(dx, O.layernorm_backward(x.double(), dy.double(), gamma.double()), rtol, scale=2.0, what="dx")
        assert N.plan(N.WL_LAYERNORM_BACKWARD, rows, cols, code, dict(opts, cluster_size=cluster_size)).threads == 352
    if dtype == torch.float32:
        rows, cols = 64, 8192
        x, dy, gamma = W.make_layernorm_inputs(rows, cols, "cpu", seed=5)
        x = (1000.0 + 0.01 * torch.randn(rows, cols, generator=torch.Generator().manual_seed(9))).float()
        (dx,) = try_run("layernorm_backward", (x, dy, gamma), cluster_size, opts)
        want = O.layernorm_backward(x.double(), dy.double(), gamma.double())
        # dx ~ 1 / std = 100 here; fp32 x carries 6e-5 of rounding on a spread of 1e-2, which the
        # oracle sees too (same inputs), so the usual bound holds at that scale
        close(dx, want, 2e-3, scale=float(want.abs().max()), what="dx far from zero")


@pytest.mark.parametrize("cluster_size", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("threads", [608, 352])
def test_layernorm_backward_stats_dx_only_warp_specialised_kernel(threads, dtype, cluster_size):
    opts = {"threads": threads}
    for rows, cols in ((3100, 4096), (2999, 1096)):
        inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=rows, dtype=dtype)
        dev_inputs = to_dev(inputs)
        dx = torch.empty_like(dev_inputs[0])
        try:
            L.launch_layernorm_backward_stats(dev_inputs, (dx,), cluster_size, opts)
        except N.UnsupportedShape:
            continue
        torch.cuda.synchronize()
        want_dx, _, _ = O.layernorm_backward_stats(*inputs, dtype=torch.float64)
        close(dx.cpu(), want_dx, BF16_RTOL if dtype == torch.bfloat16 else FP32_RTOL, scale=2.0, what="dx")


def test_layernorm_backward_stats_automatic_plan_is_warp_specialised():
    plan = N.plan(N.WL_LAYERNORM_BACKWARD_STATS, 8192, 65536, N.BF16)
    assert (plan.threads, plan.cluster_size, plan.vectors_per_thread, plan.full_tiles) == (352, 8, 4, 1)
    assert plan.stages == 6 and plan.smem_bytes == 22528 + 6 * 32768
    # the reference's own workload at its largest sweep shape, and dx only with given statistics
    plan = N.plan(N.WL_LAYERNORM_BACKWARD, 2048, 65536, N.F32)
    assert (plan.threads, plan.cluster_size, plan.stages) == (352, 8, 3)   # 16 never replaces an 8 that fits
    # the smallest cluster whose ring has four stages; short slices keep to half of the shared memory
    plan = N.plan(N.WL_LAYERNORM_BACKWARD, 2048, 8192, N.F32)
    assert (plan.cluster_size, plan.stages) == (2, 6)
    plan = N.plan(N.WL_LAYERNORM_FORWARD, 4096, 4096, N.BF16)
    assert (plan.cluster_size, plan.stages) == (1, 8) and plan.smem_bytes <= 113 * 1024
    # the forward kernels at their target shapes: same pipeline
    plan = N.plan(N.WL_LAYERNORM_FORWARD, 4096, 131072, N.BF16)
    assert (plan.threads, plan.cluster_size, plan.vectors_per_thread) == (352, 8, 8)
    assert N.plan(N.WL_RMSNORM_FORWARD, 1024, 32768, N.BF16).threads == 352
    # fp32 RMSNorm: the lock-step register kernel, smallest cluster whose slice fits 512 threads
    plan = N.plan(N.WL_RMSNORM_FORWARD, 1024, 32768, N.F32)
    assert (plan.threads, plan.cluster_size, plan.vectors_per_thread) == (512, 4, 4)
    # explicit thread counts keep the lock-step register kernels
    assert N.plan(N.WL_LAYERNORM_BACKWARD_STATS, 8192, 65536, N.BF16, {"threads": 512}).threads == 512


def test_python_restatement_of_the_planner_rule_matches_the_library():
    """cost_model.ws_plan_rule against credit_plan over the sweep shapes and the target shapes."""
    from credit_b200 import cost_model

    cases = [("layernorm_backward", N.WL_LAYERNORM_BACKWARD, 2048, N.F32, 2, False),
             ("layernorm_forward", N.WL_LAYERNORM_FORWARD, 4096, N.BF16, 1, False),
             ("layernorm_backward_stats", N.WL_LAYERNORM_BACKWARD_STATS, 8192, N.BF16, 2, True),
             ("rmsnorm_forward", N.WL_RMSNORM_FORWARD, 1024, N.BF16, 1, False),
             ("weighted_var_backward", N.WL_WEIGHTED_VAR_BACKWARD, 4096, N.F32, 3, False),
             ("pearson_backward", N.WL_PEARSON_BACKWARD, 4096, N.F32, 2, False),
             ("softmax_logits_backward", N.WL_SOFTMAX_LOGITS_BACKWARD, 4096, N.F32, 2, False),
             ("lars_momentum", N.WL_LARS_MOMENTUM, 4096, N.F32, 3, False),
             ("rowwise_quant", N.WL_ROWWISE_QUANT, 4096, N.F32, 1, False)]
    for name, wl, rows, dtype, arrays_in, sums in cases:
        for cols in (4096, 8192, 16384, 32768, 65536, 131072):
            want = cost_model.ws_plan_rule(name, cols, 2 if dtype == N.BF16 else 4, arrays_in, column_sums=sums)
            try:
                plan = N.plan(wl, rows, cols, dtype)
            except N.UnsupportedShape:
                assert want is None, (name, cols)
                continue
            if want is None:
                assert plan.threads != 352, (name, cols)      # the library fell back to another kernel
            else:
                assert (plan.threads, plan.cluster_size, plan.stages) == (352,) + want, (name, cols)


def test_layernorm_backward_stats_headline_width():
    rows, cols = 40, 65536
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=0)
    for p in (4, 8, 16):
        check_backward_stats(inputs, try_run("layernorm_backward_stats", inputs, p), BF16_RTOL)


def test_layernorm_backward_stats_dx_only():
    rows, cols = 50, 4096
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=8)
    dev_inputs = to_dev(inputs)
    dx = torch.empty_like(dev_inputs[0])
    L.launch_layernorm_backward_stats(dev_inputs, (dx,), 4)
    torch.cuda.synchronize()
    want_dx, _, _ = O.layernorm_backward_stats(*inputs, dtype=torch.float64)
    close(dx.cpu(), want_dx, BF16_RTOL, scale=2.0, what="dx")


def test_layernorm_backward_stats_is_deterministic():
    rows, cols = 900, 8192
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=2)
    a = run("layernorm_backward_stats", inputs, 8)
    b = run("layernorm_backward_stats", inputs, 8)
    assert all(torch.equal(p, q) for p, q in zip(a, b))


# ---------------------------------------------------------------------------
# Generic shared-memory kernels on aligned rows (the register path switched off),
# and plans that land on each path
# ---------------------------------------------------------------------------
GENERIC = {"flags": N.FLAG_NO_REGISTER_PATH}


@pytest.mark.parametrize("cluster_size", [1, 2, 8, 16])
def test_generic_path_on_aligned_rows(cluster_size):
    rows, cols = 300, 4096
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=31)
    (y,) = try_run("rmsnorm_forward", (x, gamma), cluster_size, GENERIC)
    close(y, O.rmsnorm_forward(x, gamma, dtype=torch.float64), FP32_RTOL, what="y")

    inputs = W.make_layernorm_forward_inputs(rows, cols, "cpu", seed=32)
    check_layernorm_forward(inputs, try_run("layernorm_forward", inputs, cluster_size, GENERIC), BF16_RTOL)

    inputs = W.make_layernorm_inputs(rows, cols, "cpu", seed=33)
    (dx,) = try_run("layernorm_backward", inputs, cluster_size, GENERIC)
    close(dx, O.layernorm_backward(*[t.double() for t in inputs]), FP32_RTOL, scale=2.0, what="dx")

    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=34)
    check_backward_stats(inputs, try_run("layernorm_backward_stats", inputs, cluster_size, GENERIC),
                         BF16_RTOL)


def test_generic_path_persistent_ring():
    rows, cols = 2500, 2048
    opts = dict(GENERIC, schedule=N.SCHEDULE_PERSISTENT, stages=3)
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=35)
    (y,) = run("rmsnorm_forward", (x, gamma), 2, opts)
    close(y, O.rmsnorm_forward(x, gamma, dtype=torch.float64), FP32_RTOL, what="y")


@pytest.mark.parametrize("shape", [(9, 4096), (5, 1000), (3, 1)])
def test_block_read_variant(shape):
    """One CTA per row, every pass from global memory: same results as the staged kernels."""
    rows, cols = shape
    opts = {"variant": N.VARIANT_BLOCK_READ}
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=51)
    (y,) = run("rmsnorm_forward", (x, gamma), 0, opts)
    close(y, O.rmsnorm_forward(x, gamma, dtype=torch.float64), FP32_RTOL, what="y")
    inputs = W.make_layernorm_forward_inputs(rows, cols, "cpu", seed=52)
    check_layernorm_forward(inputs, run("layernorm_forward", inputs, 0, opts), BF16_RTOL)
    inputs = W.make_layernorm_inputs(rows, cols, "cpu", seed=53)
    (dx,) = run("layernorm_backward", inputs, 0, opts)
    close(dx, O.layernorm_backward(*[t.double() for t in inputs]), FP32_RTOL, scale=2.0, what="dx")
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=54)
    check_backward_stats(inputs, run("layernorm_backward_stats", inputs, 0, opts), BF16_RTOL)
    assert N.plan(N.WL_RMSNORM_FORWARD, rows, cols, N.F32, opts).cluster_size == 1
    with pytest.raises(N.UnsupportedShape):
        N.plan(N.WL_ROW_REDUCE, rows, cols, N.F32, opts)


def test_plans_choose_the_expected_path():
    # aligned rows: register path; the flag or a ragged width: generic path
    assert N.plan(N.WL_RMSNORM_FORWARD, 1024, 32768, N.F32).vectors_per_thread > 0
    assert N.plan(N.WL_RMSNORM_FORWARD, 1024, 32768, N.F32, GENERIC).vectors_per_thread == 0
    assert N.plan(N.WL_RMSNORM_FORWARD, 8, 1001, N.F32).vectors_per_thread == 0
    assert N.plan(N.WL_LAYERNORM_FORWARD, 4096, 131072, N.BF16).vectors_per_thread > 0
    # a slice too wide for the registers of one CTA falls back to the generic kernel
    p = N.plan(N.WL_LAYERNORM_BACKWARD_STATS, 64, 65536, N.BF16, {"cluster_size": 2})
    assert p.vectors_per_thread == 0 and p.kernel_launches == 3


def test_wide_slice_column_sums_use_the_fallback_kernels():
    rows, cols = 300, 16384
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=36)
    check_backward_stats(inputs, try_run("layernorm_backward_stats", inputs, 1), BF16_RTOL)


@pytest.mark.parametrize("threads", [256, 512])
@pytest.mark.parametrize("cluster_size", [1, 2, 4, 8, 16])
def test_register_path_every_vector_count(cluster_size, threads):
    """Sweeps vectors-per-thread 1..8 through the cluster size at a fixed width."""
    rows, cols = 700, 8192
    opts = {"threads": threads}
    x, gamma = W.make_rmsnorm_inputs(rows, cols, "cpu", seed=41)
    (y,) = try_run("rmsnorm_forward", (x, gamma), cluster_size, opts)
    close(y, O.rmsnorm_forward(x, gamma, dtype=torch.float64), FP32_RTOL, what="y")
    inputs = W.make_layernorm_forward_inputs(rows, cols, "cpu", seed=42, dtype=torch.float32)
    check_layernorm_forward(inputs, try_run("layernorm_forward", inputs, cluster_size, opts), FP32_RTOL)
    inputs = W.make_layernorm_inputs(rows, cols, "cpu", seed=43)
    (dx,) = try_run("layernorm_backward", inputs, cluster_size, opts)
    close(dx, O.layernorm_backward(*[t.double() for t in inputs]), FP32_RTOL, scale=2.0, what="dx")


# ---------------------------------------------------------------------------
# Argument checking and the launch plan
# ---------------------------------------------------------------------------
def test_bad_arguments_are_reported_not_fatal():
    x, gamma = to_dev(W.make_rmsnorm_inputs(4, 256, "cpu"))
    y = torch.empty_like(x)
    with pytest.raises(N.CreditError) as err:
        L.launch_rmsnorm_forward((x, gamma), (y,), 3)
    assert err.value.code == N.ERR_INVALID_ARGUMENT and "cluster_size" in err.value.message
    with pytest.raises(N.CreditError):
        L.launch_rmsnorm_forward((x, gamma), (y,), 0, {"threads": 100})
    with pytest.raises(N.UnsupportedShape):
        # 4 MiB rows cannot be staged by one CTA
        N.plan(N.WL_RMSNORM_FORWARD, 8, 1 << 20, N.F32, {"variant": N.VARIANT_BLOCK_SMEM})
    with pytest.raises(ValueError):
        L.launch_rmsnorm_forward((x.cpu(), gamma), (y,))
    # rings deeper than 8 stages belong to the warp-specialised kernels only; 17 is too deep for any
    with pytest.raises(N.UnsupportedShape):
        N.plan(N.WL_RMSNORM_FORWARD, 64, 4096, N.F32, {"threads": 512, "stages": 12})
    with pytest.raises(N.UnsupportedShape):
        N.plan(N.WL_ROW_REDUCE, 64, 65536, N.F32, {"load_path": N.LOAD_TMA, "stages": 12})
    assert N.plan(N.WL_RMSNORM_FORWARD, 64, 4096, N.F32, {"threads": 352, "stages": 12}).stages == 12
    with pytest.raises(N.CreditError):
        N.plan(N.WL_RMSNORM_FORWARD, 64, 4096, N.F32, {"stages": 17})
    code = N.load().credit_rmsnorm_forward(None, None, None, 1, 1, 1e-6, 0, None, None)
    assert code == N.ERR_INVALID_ARGUMENT
    # the library still works after failures
    L.launch_rmsnorm_forward((x, gamma), (y,), 2)
    torch.cuda.synchronize()


def test_workspace_too_small_is_rejected():
    inputs = to_dev(W.make_layernorm_backward_stats_inputs(64, 2048, "cpu"))
    outs = L.allocate_outputs("layernorm_backward_stats", inputs)
    tiny = torch.empty(64, dtype=torch.uint8, device=DEV)
    with pytest.raises(N.CreditError) as err:
        L.launch_layernorm_backward_stats(inputs, outs, 2, None, workspace=tiny)
    assert err.value.code == N.ERR_WORKSPACE


def test_empty_batch_is_a_no_op():
    x = torch.empty(0, 512, device=DEV)
    gamma = torch.ones(512, device=DEV)
    y = torch.empty_like(x)
    L.launch_rmsnorm_forward((x, gamma), (y,))
    s = torch.empty(0, device=DEV)
    L.launch_row_reduce((x,), (s, s.clone(), torch.empty(0, device=DEV, dtype=torch.int64)))
    torch.cuda.synchronize()


def test_plan_and_device_query():
    info = N.query_device()
    assert info.sm_major == 10 and info.cluster_launch == 1
    assert info.max_dynamic_smem_per_block >= 200 * 1024
    p = N.plan(N.WL_LAYERNORM_BACKWARD_STATS, 8192, 65536, N.BF16)
    assert p.cluster_size in (4, 8, 16) and p.aligned == 1 and p.vectors_per_thread in (1, 2, 4)
    assert p.workspace_bytes == p.num_clusters * 2 * 65536 * 4
    assert p.grid_ctas == p.num_clusters * p.cluster_size
    p = N.plan(N.WL_ROW_REDUCE, 512, 1 << 20, N.F32)
    assert p.smem_bytes <= info.max_dynamic_smem_per_block


def test_credit_bench_times_every_workload():
    """The self-contained timing entry point: positive times, n/a reported as UNSUPPORTED."""
    import ctypes
    lib = N.load()
    ms = ctypes.c_double(0.0)
    names = ["rmsnorm_forward", "row_reduce", "layernorm_forward", "layernorm_backward", "layernorm_backward_stats",
             "weighted_var_backward", "pearson_backward", "softmax_logits_backward", "lars_momentum", "rowwise_quant"]
    for name in names:
        for cluster, variant in ((0, N.VARIANT_AUTO), (4, N.VARIANT_CLUSTER_SMEM)):
            rc = lib.credit_bench(name.encode(), 64, 8192, N.F32, cluster, variant, 2, 3, ctypes.byref(ms))
            assert rc == N.CREDIT_OK, (name, cluster, lib.credit_last_error())
            assert 0.0 < ms.value < 50.0
    assert lib.credit_bench(b"layernorm_forward", 64, 8192, N.BF16, 8, N.VARIANT_CLUSTER_SMEM, 1, 2,
                            ctypes.byref(ms)) == N.CREDIT_OK
    # a staged single-CTA variant cannot hold a 1M-column row
    assert lib.credit_bench(b"rmsnorm_forward", 4, 1048576, N.F32, 0, N.VARIANT_BLOCK_SMEM, 1, 1,
                            ctypes.byref(ms)) == N.ERR_UNSUPPORTED
    assert lib.credit_bench(b"no_such_workload", 4, 64, N.F32, 0, 0, 1, 1, ctypes.byref(ms)) == N.ERR_INVALID_ARGUMENT
    assert lib.credit_bench(b"row_reduce", 4, 64, N.BF16, 0, 0, 1, 1, ctypes.byref(ms)) == N.ERR_INVALID_ARGUMENT


def test_runner_in_process_arm():
    from credit_b200 import runner

    res = runner.benchmark_native("layernorm_backward", 128, 8192, warmup=2, iterations=5, trials=2, cluster_size=4)
    assert res["framework"] == "native" and 0.0 < res["ms"] < 10.0 and len(res["samples"]) == 2
    res = runner.benchmark_native("rowwise_quant", 64, 4096, warmup=1, iterations=3, trials=1)
    assert res["gbps"] > 0.0


@pytest.mark.parametrize("cluster_size", [0, 1, 2, 4, 8, 16])
def test_layernorm_backward_reproduces_reference_outputs(cluster_size):
    """dx on the stored golden inputs against what the reference's own function returned."""
    import numpy as np
    from pathlib import Path

    golden = np.load(Path(__file__).resolve().parent / "golden" / "reference_workloads.npz")
    for shape in ("3x96", "2x1000"):
        ins = tuple(torch.from_numpy(golden[f"layernorm_backward/{shape}/in{i}"]) for i in range(3))
        want = torch.from_numpy(golden[f"layernorm_backward/{shape}/out0"])
        (got,) = try_run("layernorm_backward", ins, cluster_size)
        # same formula in fp32 on both sides: rounding noise only (the reference's own gate is 2e-2)
        assert torch.allclose(got, want, rtol=1e-4, atol=2e-5), float((got - want).abs().max())
