"""The LayerNorm-backward entry point that brings its own scratch memory.

Some callers may not allocate device memory at the moment they need the kernel
(a serving loop that must not stall on the allocator, a host application that
gives a plug-in no allocator). `credit_layernorm_backward_stats_static` serves
them from a fixed array inside the library. This file checks, through the C ABI,
that it returns what the workspace-taking entry point returns, twice in a row
(the array is shared between calls and keeps its old contents), and that it
refuses shapes that do not fit. It is named to be collected after every other
test file, and it needs nothing from them.
"""
import ctypes

import pytest
import torch

from credit_b200 import _native as N
from credit_b200 import launchers as L
from credit_b200 import workloads as W

pytestmark = pytest.mark.gpu

FP32_RTOL = 1.0e-5
BF16_RTOL = 2.0e-2


def _close(got, want, rtol, scale):
    err = (got.double() - want.double()).abs()
    assert bool((err <= rtol * want.double().abs() + rtol * scale).all()), float(err.max())


def _call_static(lib, inputs, outputs, opts=None):
    x, dy, gamma, mean, rstd = inputs
    dx, dgamma, dbeta = outputs
    rows, cols = x.shape
    dtype = N.BF16 if x.dtype == torch.bfloat16 else N.F32
    code = lib.credit_layernorm_backward_stats_static(
        x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
        dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), rows, cols, dtype, N.opts_ref(opts),
        torch.cuda.current_stream().cuda_stream)
    N.check(code)


@pytest.mark.parametrize("shape,dtype", [((300, 4096), torch.bfloat16), ((65, 1000), torch.float32)])
def test_static_scratch_matches_the_workspace_entry_point_twice(native_lib, shape, dtype):
    dev = torch.device("cuda:0")
    rows, cols = shape
    inputs = tuple(t.to(dev) for t in
                   W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=5, dtype=dtype))
    want = L.allocate_outputs("layernorm_backward_stats", inputs)
    L.launch_layernorm_backward_stats(inputs, want)          # existing entry point, torch workspace
    torch.cuda.synchronize()
    rtol_dx = BF16_RTOL if dtype == torch.bfloat16 else FP32_RTOL
    for call in range(2):
        got = L.allocate_outputs("layernorm_backward_stats", inputs)
        for t in got:
            t.fill_(float("nan"))
        _call_static(native_lib, inputs, got)
        torch.cuda.synchronize()
        _close(got[0].cpu(), want[0].cpu(), rtol_dx, 2.0)
        _close(got[1].cpu(), want[1].cpu(), FP32_RTOL, 4.0 * rows ** 0.5)
        _close(got[2].cpu(), want[2].cpu(), FP32_RTOL, 4.0 * rows ** 0.5)
    assert N.device_status() == 0


def test_static_scratch_refuses_shapes_beyond_its_capacity(native_lib):
    capacity = native_lib.credit_layernorm_backward_stats_static_capacity()
    assert capacity == 16 << 20
    rows, cols = 4096, 262144
    need = native_lib.credit_layernorm_backward_stats_workspace_bytes(rows, cols, N.BF16, None)
    assert need > capacity
    # refused on size alone: no pointer is touched, so none is needed here
    code = native_lib.credit_layernorm_backward_stats_static(
        None, None, None, None, None, None, None, None, rows, cols, N.BF16, None, None)
    assert code == N.ERR_WORKSPACE
    assert "built-in scratch" in N.last_error()
