"""Host-buffer calls: the workloads on tensors that live in (pinned) HOST memory.

Thin wrappers over the `credit_*_host` entry points of the C ABI: inputs and outputs
are CPU tensors, `scratch` is a uint8 CUDA tensor of at least `scratch_bytes(...)`
bytes that the library streams row blocks through (upload, kernels and download of
neighbouring blocks overlap). A call returns when its results are in host memory.
This is the end-to-end path `bench.py` times as `e2e`; the reference's counterpart is
`run_shape` in its executables (`src/workloads/layernorm_backward.cu:767-805`), which
own their device buffers.
"""
from __future__ import annotations

import torch

from . import _native as N


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return N.F32
    if t.dtype == torch.bfloat16:
        return N.BF16
    raise TypeError(f"unsupported dtype {t.dtype}")


def _host(name: str, t: torch.Tensor, dtype=None, shape=None) -> int:
    if t.device.type != "cpu" or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous CPU tensor")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    return t.data_ptr()


def _scratch(scratch: torch.Tensor) -> tuple[int, int]:
    if scratch.device.type != "cuda" or scratch.dtype != torch.uint8 or not scratch.is_contiguous():
        raise ValueError("scratch must be a contiguous uint8 CUDA tensor")
    return scratch.data_ptr(), scratch.numel()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def scratch_bytes(workload: str, rows: int, cols: int, dtype: torch.dtype = torch.float32, hidden: int = 0) -> int:
    """Minimum scratch of a host call; more lets the row blocks grow (up to the whole matrix)."""
    lib = N.load()
    code = N.BF16 if dtype == torch.bfloat16 else N.F32
    if workload == "row_reduce":
        return lib.credit_row_reduce_host_scratch_bytes(rows, cols)
    if workload == "rmsnorm_forward":
        return lib.credit_rmsnorm_forward_host_scratch_bytes(rows, cols, code)
    if workload == "layernorm_forward":
        return lib.credit_layernorm_forward_host_scratch_bytes(rows, cols, code)
    if workload == "layernorm_backward_stats":
        return lib.credit_layernorm_backward_stats_host_scratch_bytes(rows, cols, code, None)
    if workload == "ffn_forward":
        return lib.credit_ffn_forward_host_scratch_bytes(rows, cols, hidden)
    raise KeyError(workload)


def row_reduce(x, out_sum, out_max, out_argmax, scratch, opts=None) -> None:
    rows, cols = x.shape
    sp, sn = _scratch(scratch)
    N.check(N.load().credit_row_reduce_host(
        _host("x", x, torch.float32), _host("sum", out_sum, torch.float32, (rows,)),
        _host("max", out_max, torch.float32, (rows,)), _host("argmax", out_argmax, torch.int64, (rows,)),
        rows, cols, N.opts_ref(opts), sp, sn, _stream()))


def rmsnorm_forward(x, gamma, y, scratch, eps: float = 1.0e-6, opts=None) -> None:
    rows, cols = x.shape
    sp, sn = _scratch(scratch)
    N.check(N.load().credit_rmsnorm_forward_host(
        _host("x", x), _host("gamma", gamma, torch.float32, (cols,)), _host("y", y, x.dtype, x.shape),
        rows, cols, eps, _dtype_code(x), N.opts_ref(opts), sp, sn, _stream()))


def layernorm_forward(x, gamma, beta, y, mean, rstd, scratch, eps: float = 1.0e-5, opts=None) -> None:
    rows, cols = x.shape
    sp, sn = _scratch(scratch)
    N.check(N.load().credit_layernorm_forward_host(
        _host("x", x), _host("gamma", gamma, torch.float32, (cols,)), _host("beta", beta, torch.float32, (cols,)),
        _host("y", y, x.dtype, x.shape), _host("mean", mean, torch.float32, (rows,)),
        _host("rstd", rstd, torch.float32, (rows,)), rows, cols, eps, _dtype_code(x), N.opts_ref(opts), sp, sn,
        _stream()))


def layernorm_backward_stats(x, dy, gamma, mean, rstd, dx, dgamma, dbeta, scratch, opts=None) -> None:
    rows, cols = x.shape
    sp, sn = _scratch(scratch)
    N.check(N.load().credit_layernorm_backward_stats_host(
        _host("x", x), _host("dy", dy, x.dtype, x.shape), _host("gamma", gamma, torch.float32, (cols,)),
        _host("mean", mean, torch.float32, (rows,)), _host("rstd", rstd, torch.float32, (rows,)),
        _host("dx", dx, x.dtype, x.shape), _host("dgamma", dgamma, torch.float32, (cols,)),
        _host("dbeta", dbeta, torch.float32, (cols,)), rows, cols, _dtype_code(x), N.opts_ref(opts), sp, sn,
        _stream()))


def ffn_forward(x, w1_packed, w2_packed, gamma, y, scratch, eps: float = 1.0e-6) -> None:
    """x, y: bf16 [m, d] on the host; w1_packed [h, d], w2_packed [d, h] and gamma [d] on the device."""
    m, d = x.shape
    h = w1_packed.shape[0]
    for name, t in (("w1_packed", w1_packed), ("w2_packed", w2_packed), ("gamma", gamma)):
        if t.device.type != "cuda" or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CUDA tensor")
    sp, sn = _scratch(scratch)
    N.check(N.load().credit_ffn_forward_host(
        _host("x", x, torch.bfloat16), w1_packed.data_ptr(), w2_packed.data_ptr(), gamma.data_ptr(),
        _host("y", y, torch.bfloat16, x.shape), m, d, h, eps, sp, sn, _stream()))
