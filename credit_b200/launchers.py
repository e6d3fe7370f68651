"""In-process launcher table of the native backend.

Same convention as the reference's Triton table
(`dsmem_eval/triton_kernels.py:300-414`): `launcher(inputs, outputs, ...)`
takes caller-owned device tensors, enqueues on the current CUDA stream and
returns nothing; `allocate_outputs(name, inputs)` pre-allocates the outputs. The
Triton knobs (`block_size`, `num_warps`) have no meaning for these kernels; the
knobs here are the cluster size and the other launch options of the C ABI.

torch is used for device memory and streams only; every kernel is in
`libcredit_b200.so`.
"""
from __future__ import annotations

import torch

from . import _native as N

_DTYPES = {torch.float32: N.F32, torch.bfloat16: N.BF16}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check_matrix(name: str, t: torch.Tensor, dtype=None, shape=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


def _row_dtype(x: torch.Tensor) -> int:
    if x.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {x.dtype}: float32 and bfloat16 only")
    return _DTYPES[x.dtype]


def _opts(cluster_size: int, opts) -> "N.LaunchOpts | None":
    o = N.make_opts(opts)
    if cluster_size:
        if o is None:
            o = N.LaunchOpts()
        else:
            o = N.LaunchOpts(**{name: getattr(o, name) for name, _ in N.LaunchOpts._fields_})
        o.cluster_size = int(cluster_size)
    return o


def _ref(o):
    import ctypes
    return None if o is None else ctypes.byref(o)


def launch_rmsnorm_forward(inputs, outputs, cluster_size: int = 0, opts=None, eps: float = 1.0e-6) -> None:
    x, gamma = inputs
    (y,) = outputs
    _check_matrix("x", x)
    rows, cols = x.shape
    _check_matrix("gamma", gamma, torch.float32, (cols,))
    _check_matrix("y", y, x.dtype, x.shape)
    o = _opts(cluster_size, opts)
    with torch.cuda.device(x.device):
        N.check(N.load().credit_rmsnorm_forward(
            x.data_ptr(), gamma.data_ptr(), y.data_ptr(), rows, cols, eps, _row_dtype(x), _ref(o),
            _stream_ptr()))


def launch_row_reduce(inputs, outputs, cluster_size: int = 0, opts=None) -> None:
    (x,) = inputs
    row_sum, row_max, row_argmax = outputs
    _check_matrix("x", x, torch.float32)
    rows, cols = x.shape
    _check_matrix("sum", row_sum, torch.float32, (rows,))
    _check_matrix("max", row_max, torch.float32, (rows,))
    _check_matrix("argmax", row_argmax, torch.int64, (rows,))
    o = _opts(cluster_size, opts)
    with torch.cuda.device(x.device):
        N.check(N.load().credit_row_reduce(
            x.data_ptr(), row_sum.data_ptr(), row_max.data_ptr(), row_argmax.data_ptr(), rows, cols,
            _ref(o), _stream_ptr()))


def launch_layernorm_forward(inputs, outputs, cluster_size: int = 0, opts=None, eps: float = 1.0e-5) -> None:
    x, gamma, beta = inputs
    y, mean, rstd = outputs
    _check_matrix("x", x)
    rows, cols = x.shape
    _check_matrix("gamma", gamma, torch.float32, (cols,))
    _check_matrix("beta", beta, torch.float32, (cols,))
    _check_matrix("y", y, x.dtype, x.shape)
    _check_matrix("mean", mean, torch.float32, (rows,))
    _check_matrix("rstd", rstd, torch.float32, (rows,))
    o = _opts(cluster_size, opts)
    with torch.cuda.device(x.device):
        N.check(N.load().credit_layernorm_forward(
            x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), mean.data_ptr(),
            rstd.data_ptr(), rows, cols, eps, _row_dtype(x), _ref(o), _stream_ptr()))


def launch_layernorm_backward(inputs, outputs, cluster_size: int = 0, opts=None, eps: float = 1.0e-5) -> None:
    """dx with statistics recomputed from x: the reference workload
    (`launch_layernorm_backward`, triton_kernels.py:300-312)."""
    x, dy, gamma = inputs
    (dx,) = outputs
    _check_matrix("x", x)
    rows, cols = x.shape
    _check_matrix("dy", dy, x.dtype, x.shape)
    _check_matrix("gamma", gamma, torch.float32, (cols,))
    _check_matrix("dx", dx, x.dtype, x.shape)
    o = _opts(cluster_size, opts)
    with torch.cuda.device(x.device):
        N.check(N.load().credit_layernorm_backward(
            x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), dx.data_ptr(), rows, cols, eps,
            _row_dtype(x), _ref(o), _stream_ptr()))


def layernorm_backward_stats_workspace_bytes(rows: int, cols: int, dtype: torch.dtype,
                                             cluster_size: int = 0, opts=None) -> int:
    o = _opts(cluster_size, opts)
    # credit_plan raises with the precise status if the shape or options are unusable
    N.plan(N.WL_LAYERNORM_BACKWARD_STATS, rows, cols, _DTYPES[dtype], o)
    return int(N.load().credit_layernorm_backward_stats_workspace_bytes(
        rows, cols, _DTYPES[dtype], _ref(o)))


def launch_layernorm_backward_stats(inputs, outputs, cluster_size: int = 0, opts=None,
                                    workspace: torch.Tensor | None = None) -> None:
    """dx, dgamma, dbeta from x, dy, gamma and the saved fp32 mean/rstd. `workspace` is a
    uint8 CUDA tensor of at least `layernorm_backward_stats_workspace_bytes(...)` bytes; when
    omitted one is allocated through torch's caching allocator for this call."""
    x, dy, gamma, mean, rstd = inputs
    if len(outputs) == 1:
        (dx,), dgamma, dbeta = outputs, None, None
    else:
        dx, dgamma, dbeta = outputs
    _check_matrix("x", x)
    rows, cols = x.shape
    _check_matrix("dy", dy, x.dtype, x.shape)
    _check_matrix("gamma", gamma, torch.float32, (cols,))
    _check_matrix("mean", mean, torch.float32, (rows,))
    _check_matrix("rstd", rstd, torch.float32, (rows,))
    _check_matrix("dx", dx, x.dtype, x.shape)
    o = _opts(cluster_size, opts)
    ws_ptr, ws_bytes = 0, 0
    if dgamma is not None:
        _check_matrix("dgamma", dgamma, torch.float32, (cols,))
        _check_matrix("dbeta", dbeta, torch.float32, (cols,))
        if workspace is None:
            need = layernorm_backward_stats_workspace_bytes(rows, cols, x.dtype, 0, o)
            workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
        _check_matrix("workspace", workspace, torch.uint8)
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel()
    with torch.cuda.device(x.device):
        N.check(N.load().credit_layernorm_backward_stats(
            x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
            dx.data_ptr(), 0 if dgamma is None else dgamma.data_ptr(),
            0 if dbeta is None else dbeta.data_ptr(), rows, cols, _row_dtype(x), _ref(o), ws_ptr,
            ws_bytes, _stream_ptr()))


def pack_ffn_weight(w: torch.Tensor) -> torch.Tensor:
    """[k, n] bf16 row-major weight -> the K-major [n, k] form the FFN GEMMs take (done once per
    weight, on the device)."""
    _check_matrix("w", w, torch.bfloat16)
    k, n = w.shape
    packed = torch.empty((n, k), dtype=torch.bfloat16, device=w.device)
    with torch.cuda.device(w.device):
        N.check(N.load().credit_ffn_pack_weight(w.data_ptr(), packed.data_ptr(), k, n, _stream_ptr()))
    return packed


def ffn_workspace_bytes(m: int, d: int, h: int) -> int:
    return int(N.load().credit_ffn_workspace_bytes(m, d, h))


def launch_ffn_forward(inputs, outputs, cluster_size: int = 0, opts=None, eps: float = 1.0e-6,
                       workspace: torch.Tensor | None = None) -> None:
    """Y = RMSNorm(GELU(X W1) W2 + X) * gamma. inputs = (x [m, d] bf16, w1_packed [h, d],
    w2_packed [d, h], gamma [d] fp32) with the weights from `pack_ffn_weight`. The cluster size
    is fixed by the width (d / 256 CTAs span a row); `cluster_size` and `opts` are accepted for
    the common launcher signature and must be left at their defaults."""
    x, w1p, w2p, gamma = inputs
    (y,) = outputs
    if cluster_size or opts:
        raise ValueError("the FFN takes no launch options: its cluster size is d / 256")
    _check_matrix("x", x, torch.bfloat16)
    m, d = x.shape
    h = w1p.shape[0]
    _check_matrix("w1_packed", w1p, torch.bfloat16, (h, d))
    _check_matrix("w2_packed", w2p, torch.bfloat16, (d, h))
    _check_matrix("gamma", gamma, torch.float32, (d,))
    _check_matrix("y", y, torch.bfloat16, (m, d))
    if workspace is None:
        workspace = torch.empty(max(ffn_workspace_bytes(m, d, h), 16), dtype=torch.uint8, device=x.device)
    _check_matrix("workspace", workspace, torch.uint8)
    with torch.cuda.device(x.device):
        N.check(N.load().credit_ffn_forward(
            x.data_ptr(), w1p.data_ptr(), w2p.data_ptr(), gamma.data_ptr(), y.data_ptr(), m, d, h, eps,
            workspace.data_ptr(), workspace.numel(), _stream_ptr()))


# name -> (workload id, staged inputs, per-row input?, row-major outputs, per-row output?)
_ROW_OPS = {
    "weighted_var_backward": (N.WL_WEIGHTED_VAR_BACKWARD, 3, False, 1, False),
    "pearson_backward": (N.WL_PEARSON_BACKWARD, 2, True, 2, False),
    "softmax_logits_backward": (N.WL_SOFTMAX_LOGITS_BACKWARD, 2, False, 1, False),
    "lars_momentum": (N.WL_LARS_MOMENTUM, 3, False, 2, False),
    "rowwise_quant": (N.WL_ROWWISE_QUANT, 1, False, 1, True),
}


def _make_row_op_launcher(name: str):
    workload, nin, has_row_in, nout, has_row_out = _ROW_OPS[name]

    def launch(inputs, outputs, cluster_size: int = 0, opts=None) -> None:
        if len(inputs) != nin + int(has_row_in) or len(outputs) != nout + int(has_row_out):
            raise ValueError(f"{name}: expected {nin + int(has_row_in)} inputs and {nout + int(has_row_out)} outputs")
        x = inputs[0]
        _check_matrix("input 0", x, torch.float32)
        rows, cols = x.shape
        for i in range(1, nin):
            _check_matrix(f"input {i}", inputs[i], torch.float32, (rows, cols))
        row_in = None
        if has_row_in:      # the reference passes it as [rows, 1]
            row_in = inputs[nin]
            if row_in.numel() != rows:
                raise ValueError(f"{name}: the per-row input must have {rows} elements")
            _check_matrix("per-row input", row_in, torch.float32)
        out_dtype = torch.int8 if name == "rowwise_quant" else torch.float32
        for i in range(nout):
            _check_matrix(f"output {i}", outputs[i], out_dtype, (rows, cols))
        row_out = None
        if has_row_out:
            row_out = outputs[nout]
            _check_matrix("per-row output", row_out, torch.float32, (rows,))
        ptr = [t.data_ptr() if rows else None for t in inputs[:nin]] + [None] * (3 - nin)
        N.check(N.load().credit_row_op(
            workload, ptr[0], ptr[1], ptr[2], row_in.data_ptr() if has_row_in and rows else None,
            outputs[0].data_ptr() if rows else None, outputs[1].data_ptr() if nout > 1 and rows else None,
            row_out.data_ptr() if has_row_out and rows else None, rows, cols, _ref(_opts(cluster_size, opts)),
            _stream_ptr()))

    launch.__name__ = f"launch_{name}"
    launch.__doc__ = (f"{name} of the reference sweep (dsmem_eval/workloads.py), fp32, through credit_row_op; "
                      "same launcher convention as the others.")
    return launch


NATIVE_LAUNCHERS = {
    "rmsnorm_forward": launch_rmsnorm_forward,
    "row_reduce": launch_row_reduce,
    "layernorm_forward": launch_layernorm_forward,
    "layernorm_backward": launch_layernorm_backward,
    "layernorm_backward_stats": launch_layernorm_backward_stats,
    "ffn_forward": launch_ffn_forward,
    **{name: _make_row_op_launcher(name) for name in _ROW_OPS},
}


def allocate_outputs(name: str, inputs: tuple[torch.Tensor, ...]) -> tuple[torch.Tensor, ...]:
    """Output tensors for one call (reference: allocate_outputs, triton_kernels.py:403-414)."""
    x = inputs[0]
    rows, cols = x.shape
    dev = x.device
    if name == "row_reduce":
        return (
            torch.empty(rows, device=dev, dtype=torch.float32),
            torch.empty(rows, device=dev, dtype=torch.float32),
            torch.empty(rows, device=dev, dtype=torch.int64),
        )
    if name == "layernorm_forward":
        return (
            torch.empty_like(x),
            torch.empty(rows, device=dev, dtype=torch.float32),
            torch.empty(rows, device=dev, dtype=torch.float32),
        )
    if name == "layernorm_backward_stats":
        return (
            torch.empty_like(x),
            torch.empty(cols, device=dev, dtype=torch.float32),
            torch.empty(cols, device=dev, dtype=torch.float32),
        )
    if name in ("rmsnorm_forward", "layernorm_backward", "ffn_forward", "weighted_var_backward",
                "softmax_logits_backward"):
        return (torch.empty_like(x),)
    if name in ("pearson_backward", "lars_momentum"):
        return (torch.empty_like(x), torch.empty_like(x))
    if name == "rowwise_quant":
        return (torch.empty(rows, cols, device=dev, dtype=torch.int8),
                torch.empty(rows, device=dev, dtype=torch.float32))
    raise KeyError(f"unknown workload {name!r}")
