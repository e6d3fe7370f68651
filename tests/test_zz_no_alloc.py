"""The LayerNorm-backward entry point that brings its own scratch memory.

Some callers may not allocate device memory at the moment they need the kernel
(a serving loop that must not stall on the allocator, a host application that
gives a plug-in no allocator). `credit_layernorm_backward_stats_static` serves
them from a fixed array inside the library. This file checks, through the C ABI,
that it returns what the workspace-taking entry point returns, twice in a row
(the array is shared between calls and keeps its old contents), that the calls
leave the amount of free device memory unchanged, and that it refuses shapes that
do not fit. It is named to be collected after every other test file, and it needs
nothing from them.
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
    # in fp32 on whatever device holds the tensors (the tolerances are 1e-5 and up)
    err = (got.float() - want.float()).abs()
    assert bool((err <= rtol * want.float().abs() + rtol * scale).all()), float(err.max())


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


# the last shape is the full LayerNorm-backward target shape (bf16 8192 x 65536): its per-cluster
# partial sums must fit the built-in array
@pytest.mark.parametrize("shape,dtype", [((300, 4096), torch.bfloat16), ((65, 1000), torch.float32),
                                         ((8192, 65536), torch.bfloat16)])
def test_static_scratch_matches_the_workspace_entry_point_twice(native_lib, shape, dtype):
    dev = torch.device("cuda:0")
    rows, cols = shape
    inputs = W.make_layernorm_backward_stats_inputs(rows, cols, dev, seed=5, dtype=dtype)
    want = L.allocate_outputs("layernorm_backward_stats", inputs)
    L.launch_layernorm_backward_stats(inputs, want)          # existing entry point, torch workspace
    torch.cuda.synchronize()
    rtol_dx = BF16_RTOL if dtype == torch.bfloat16 else FP32_RTOL
    got = [L.allocate_outputs("layernorm_backward_stats", inputs) for _ in range(2)]
    # The first call on a device may load the library's device code (the built-in array is part
    # of it); free memory is compared from after that point on, around the two calls alone
    # (torch's own allocator is not used between the two readings).
    _call_static(native_lib, inputs, got[0])
    for outs in got:
        for t in outs:
            t.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    for outs in got:
        _call_static(native_lib, inputs, outs)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before, "the calls changed the amount of free device memory"
    for outs in got:   # compared on the device: the large shape is 1 GiB per tensor
        _close(outs[0], want[0], rtol_dx, 2.0)
        _close(outs[1], want[1], FP32_RTOL, 4.0 * rows ** 0.5)
        _close(outs[2], want[2], FP32_RTOL, 4.0 * rows ** 0.5)
    assert N.device_status() == 0


def test_static_scratch_without_column_sums_needs_no_scratch(native_lib):
    """dgamma = dbeta = NULL: dx only, no size check (nothing is written to the array)."""
    dev = torch.device("cuda:0")
    rows, cols = 40, 8192
    inputs = tuple(t.to(dev) for t in W.make_layernorm_backward_stats_inputs(rows, cols, "cpu", seed=6))
    want = L.allocate_outputs("layernorm_backward_stats", inputs)
    L.launch_layernorm_backward_stats(inputs, want)
    x, dy, gamma, mean, rstd = inputs
    dx = torch.full_like(want[0], float("nan"))
    N.check(native_lib.credit_layernorm_backward_stats_static(
        x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
        None, None, rows, cols, N.BF16, None, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    _close(dx, want[0], BF16_RTOL, 2.0)


def test_static_scratch_refuses_shapes_beyond_its_capacity(native_lib):
    capacity = native_lib.credit_layernorm_backward_stats_static_capacity()
    assert capacity == 16 << 20
    rows, cols = 4096, 262144
    need = native_lib.credit_layernorm_backward_stats_workspace_bytes(rows, cols, N.BF16, None)
    assert need > capacity
    # refused on size alone, before any pointer is dereferenced: a small buffer stands in for all
    # of them (16-byte aligned, like real inputs; column sums requested)
    stand_in = torch.empty(64, dtype=torch.float32, device="cuda:0")
    p = stand_in.data_ptr()
    code = native_lib.credit_layernorm_backward_stats_static(
        p, p, p, p, p, p, p, p, rows, cols, N.BF16, None, None)
    assert code == N.ERR_WORKSPACE
    assert "built-in scratch" in N.last_error()
