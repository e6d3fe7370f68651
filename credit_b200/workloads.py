"""Workload registry: names, shapes, seeded input factories and traffic metadata.

Mirrors `WorkloadSpec` / `WORKLOADS` of the reference
(`dsmem_eval/workloads.py:16-37, 157-212`) and its `workload_metadata.py`. The
reference keeps an eager PyTorch function in every spec; here the CPU
restatements live outside the package (they are test infrastructure), so a spec
carries only what the native path itself needs: the input factory, the output
allocator's shapes, tolerances and the byte accounting used for GB/s.

Input factories keep the reference convention `factory(rows, cols, device)` and
draw from `torch.Generator(device).manual_seed(seed)` in a fixed order, so the
same call on the CPU always gives the same bits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

TensorTuple = tuple[torch.Tensor, ...]
InputFactory = Callable[..., TensorTuple]


@dataclass(frozen=True)
class WorkloadSpec:
    name: str
    label: str
    category: str
    rows: int                      # default row count (reference: WorkloadSpec.rows)
    cols: int                      # default row width (the headline shape)
    dtype: torch.dtype
    input_factory: InputFactory
    eps: float
    # model metadata, as in workload_metadata.py:6-35
    modeled_bytes_per_element: float   # traffic of the no-DSMEM multi-pass kernel
    reread_bytes_per_element: float    # part of it that staging removes
    staged_bytes_per_element: int      # shared memory per row element
    reductions_per_stage: tuple[int, ...]
    atol: float
    rtol: float
    # compulsory traffic of one call: every input read once, every output written once
    algorithmic_bytes: Callable[[int, int], int]

    @property
    def barrier_count(self) -> int:
        """Cluster barriers per row. The reference needs two per reduction stage
        (workloads.py:31-33); double-buffered slots make it one."""
        return len(self.reductions_per_stage)

    @property
    def partial_count(self) -> int:
        return sum(self.reductions_per_stage)


def _generator(device, seed: int) -> torch.Generator:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    return gen


def _uniform(shape, low: float, high: float, device, gen) -> torch.Tensor:
    out = torch.empty(shape, device=device, dtype=torch.float32)
    return out.uniform_(low, high, generator=gen)


def _normal(shape, mean: float, std: float, device, gen) -> torch.Tensor:
    out = torch.empty(shape, device=device, dtype=torch.float32)
    return out.normal_(mean, std, generator=gen)


def make_rmsnorm_inputs(rows: int, cols: int, device, seed: int = 0) -> TensorTuple:
    """x ~ N(0,1) fp32 [rows, cols]; gamma ~ U(0.5, 1.5) [cols]."""
    gen = _generator(device, seed)
    x = _normal((rows, cols), 0.0, 1.0, device, gen)
    gamma = _uniform((cols,), 0.5, 1.5, device, gen)
    return x, gamma


def make_row_reduce_inputs(rows: int, cols: int, device, seed: int = 0) -> TensorTuple:
    """x ~ N(0,1) fp32 with one planted +10 per row at a uniformly drawn column."""
    gen = _generator(device, seed)
    x = _normal((rows, cols), 0.0, 1.0, device, gen)
    where = torch.randint(0, cols, (rows,), device=device, generator=gen)
    x[torch.arange(rows, device=device), where] = 10.0
    return (x,)


def make_layernorm_forward_inputs(rows: int, cols: int, device, seed: int = 0,
                                  dtype: torch.dtype = torch.bfloat16) -> TensorTuple:
    """x ~ N(mean 0.5, std 2.0) rounded to `dtype`; gamma ~ U(0.5,1.5); beta ~ N(0, 0.1)."""
    gen = _generator(device, seed)
    x = _normal((rows, cols), 0.5, 2.0, device, gen).to(dtype)
    gamma = _uniform((cols,), 0.5, 1.5, device, gen)
    beta = _normal((cols,), 0.0, 0.1, device, gen)
    return x, gamma, beta


def row_statistics(x: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 mean and rstd of each row (biased variance), as a LayerNorm forward saves them."""
    xf = x.float()
    mean = xf.mean(dim=-1)
    var = (xf - mean[:, None]).square().mean(dim=-1)
    return mean, torch.rsqrt(var + eps)


def make_layernorm_backward_stats_inputs(rows: int, cols: int, device, seed: int = 0,
                                         dtype: torch.dtype = torch.bfloat16) -> TensorTuple:
    """x, dy ~ N(0,1) rounded to `dtype`; gamma ~ U(0.5,1.5); fp32 mean/rstd of x (eps 1e-5)."""
    gen = _generator(device, seed)
    x = _normal((rows, cols), 0.0, 1.0, device, gen).to(dtype)
    dy = _normal((rows, cols), 0.0, 1.0, device, gen).to(dtype)
    gamma = _uniform((cols,), 0.5, 1.5, device, gen)
    # statistics in row blocks so wide inputs do not need a full fp32 copy
    mean = torch.empty(rows, device=device, dtype=torch.float32)
    rstd = torch.empty(rows, device=device, dtype=torch.float32)
    step = max(1, (1 << 26) // max(cols, 1))
    for r0 in range(0, rows, step):
        m, r = row_statistics(x[r0:r0 + step], 1.0e-5)
        mean[r0:r0 + step] = m
        rstd[r0:r0 + step] = r
    return x, dy, gamma, mean, rstd


def make_layernorm_inputs(rows: int, cols: int, device, seed: int | None = None) -> TensorTuple:
    """The reference's LayerNorm-backward inputs (workloads.py:45-50): x, dy ~ U(-1,1),
    gamma ~ U(0.75, 1.25), fp32. With seed=None the global torch RNG is used, which is
    what the reference does after torch.manual_seed(1234 + cols) (runner.py:358)."""
    gen = None if seed is None else _generator(device, seed)
    return (
        _uniform((rows, cols), -1.0, 1.0, device, gen),
        _uniform((rows, cols), -1.0, 1.0, device, gen),
        _uniform((cols,), 0.75, 1.25, device, gen),
    )


def make_ffn_inputs(rows: int, cols: int, device, seed: int = 0, hidden: int | None = None) -> TensorTuple:
    """x ~ N(0,1) [rows, cols]; W1 ~ N(0, 0.02) [cols, hidden]; W2 ~ N(0, 0.02) [hidden, cols], all
    rounded to bf16; gamma ~ U(0.5, 1.5) fp32 [cols]. hidden defaults to 4 * cols. The weights are
    returned in their natural [k, n] layout; `launchers.pack_ffn_weight` makes the K-major copies."""
    hidden = 4 * cols if hidden is None else hidden
    gen = _generator(device, seed)
    x = _normal((rows, cols), 0.0, 1.0, device, gen).to(torch.bfloat16)
    w1 = _normal((cols, hidden), 0.0, 0.02, device, gen).to(torch.bfloat16)
    w2 = _normal((hidden, cols), 0.0, 0.02, device, gen).to(torch.bfloat16)
    gamma = _uniform((cols,), 0.5, 1.5, device, gen)
    return x, w1, w2, gamma


# Input factories of the reference sweep's other workloads (dsmem_eval/workloads.py:64-150):
# same uniform ranges, seeded like the rest of this registry.
def make_weighted_var_inputs(rows: int, cols: int, device, seed: int = 0) -> TensorTuple:
    gen = _generator(device, seed)
    return (_uniform((rows, cols), -2.0, 2.0, device, gen), _uniform((rows, cols), 0.5, 1.5, device, gen),
            _uniform((rows, cols), -1.0, 1.0, device, gen))


def make_pearson_inputs(rows: int, cols: int, device, seed: int = 0) -> TensorTuple:
    gen = _generator(device, seed)
    return (_uniform((rows, cols), -1.0, 1.0, device, gen), _uniform((rows, cols), -1.0, 1.0, device, gen),
            _uniform((rows, 1), 0.75, 1.25, device, gen))


def make_softmax_inputs(rows: int, cols: int, device, seed: int = 0) -> TensorTuple:
    gen = _generator(device, seed)
    return (_uniform((rows, cols), -4.0, 4.0, device, gen), _uniform((rows, cols), -1.0, 1.0, device, gen))


def make_lars_inputs(rows: int, cols: int, device, seed: int = 0) -> TensorTuple:
    gen = _generator(device, seed)
    return tuple(_uniform((rows, cols), -1.0, 1.0, device, gen) for _ in range(3))


def make_quant_inputs(rows: int, cols: int, device, seed: int = 0) -> TensorTuple:
    return (_uniform((rows, cols), -1.0, 1.0, device, _generator(device, seed)),)


def ffn_flops(rows: int, cols: int, hidden: int) -> int:
    return 2 * (2 * rows * cols * hidden)


def _elem(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


WORKLOADS: dict[str, WorkloadSpec] = {
    "rmsnorm_forward": WorkloadSpec(
        name="rmsnorm_forward", label="RMSNorm forward", category="normalization",
        rows=1024, cols=32768, dtype=torch.float32, input_factory=make_rmsnorm_inputs, eps=1.0e-6,
        modeled_bytes_per_element=16.0, reread_bytes_per_element=4.0, staged_bytes_per_element=4,
        reductions_per_stage=(1,), atol=1.0e-5, rtol=1.0e-5,
        algorithmic_bytes=lambda r, c: 2 * r * c * 4 + c * 4,
    ),
    "row_reduce": WorkloadSpec(
        name="row_reduce", label="Row sum / max / argmax", category="reduction",
        rows=512, cols=1048576, dtype=torch.float32, input_factory=make_row_reduce_inputs, eps=0.0,
        modeled_bytes_per_element=4.0, reread_bytes_per_element=0.0, staged_bytes_per_element=0,
        reductions_per_stage=(3,), atol=1.0e-5, rtol=1.0e-5,
        algorithmic_bytes=lambda r, c: r * c * 4 + r * 16,
    ),
    "layernorm_forward": WorkloadSpec(
        name="layernorm_forward", label="LayerNorm forward", category="normalization",
        rows=4096, cols=131072, dtype=torch.bfloat16, input_factory=make_layernorm_forward_inputs,
        eps=1.0e-5,
        modeled_bytes_per_element=16.0, reread_bytes_per_element=4.0, staged_bytes_per_element=2,
        reductions_per_stage=(2,), atol=2.0e-2, rtol=2.0e-2,
        algorithmic_bytes=lambda r, c: 2 * r * c * 2 + 2 * c * 4 + 2 * r * 4,
    ),
    "layernorm_backward": WorkloadSpec(
        name="layernorm_backward", label="LayerNorm backward", category="normalization",
        rows=2048, cols=65536, dtype=torch.float32, input_factory=make_layernorm_inputs, eps=1.0e-5,
        modeled_bytes_per_element=32.0, reread_bytes_per_element=12.0, staged_bytes_per_element=8,
        reductions_per_stage=(2, 2), atol=2.0e-2, rtol=2.0e-2,
        algorithmic_bytes=lambda r, c: 3 * r * c * 4 + c * 4,
    ),
    "layernorm_backward_stats": WorkloadSpec(
        name="layernorm_backward_stats", label="LayerNorm backward (dx, dgamma, dbeta)",
        category="normalization",
        rows=8192, cols=65536, dtype=torch.bfloat16,
        input_factory=make_layernorm_backward_stats_inputs, eps=1.0e-5,
        modeled_bytes_per_element=10.0, reread_bytes_per_element=4.0, staged_bytes_per_element=4,
        reductions_per_stage=(2,), atol=2.0e-2, rtol=2.0e-2,
        algorithmic_bytes=lambda r, c: 3 * r * c * 2 + 2 * r * 4 + c * 4 + 2 * c * 4,
    ),
    "ffn_forward": WorkloadSpec(
        name="ffn_forward", label="Fused FFN (GEMM + GELU, GEMM + residual + RMSNorm)",
        category="gemm",
        rows=2048, cols=4096, dtype=torch.bfloat16, input_factory=make_ffn_inputs, eps=1.0e-6,
        modeled_bytes_per_element=0.0, reread_bytes_per_element=0.0, staged_bytes_per_element=0,
        reductions_per_stage=(1,), atol=2.0e-2, rtol=2.0e-2,
        # compulsory bytes with hidden = 4 * cols: X, W1, W2, Y (the hidden activations stay on chip
        # only in a fully fused kernel; this implementation also writes and reads them once)
        algorithmic_bytes=lambda r, c: 2 * r * c * 2 + 2 * c * 4 * c * 2 + c * 4,
    ),
    # the rest of the reference sweep: metadata of workload_metadata.py:17-34, tolerances of
    # workloads.py:164-210
    "weighted_var_backward": WorkloadSpec(
        name="weighted_var_backward", label="Weighted variance backward", category="normalization",
        rows=4096, cols=65536, dtype=torch.float32, input_factory=make_weighted_var_inputs, eps=1.0e-5,
        modeled_bytes_per_element=40.0, reread_bytes_per_element=24.0, staged_bytes_per_element=12,
        reductions_per_stage=(2, 3), atol=3.0e-2, rtol=3.0e-2,
        algorithmic_bytes=lambda r, c: 4 * r * c * 4,
    ),
    "pearson_backward": WorkloadSpec(
        name="pearson_backward", label="Pearson backward", category="pairwise statistics",
        rows=4096, cols=65536, dtype=torch.float32, input_factory=make_pearson_inputs, eps=1.0e-6,
        modeled_bytes_per_element=24.0, reread_bytes_per_element=8.0, staged_bytes_per_element=8,
        reductions_per_stage=(2, 3), atol=3.0e-3, rtol=3.0e-3,
        algorithmic_bytes=lambda r, c: 4 * r * c * 4 + r * 4,
    ),
    "softmax_logits_backward": WorkloadSpec(
        name="softmax_logits_backward", label="Softmax-logits backward", category="softmax",
        rows=4096, cols=65536, dtype=torch.float32, input_factory=make_softmax_inputs, eps=0.0,
        modeled_bytes_per_element=28.0, reread_bytes_per_element=16.0, staged_bytes_per_element=8,
        reductions_per_stage=(1, 1, 1), atol=3.0e-3, rtol=3.0e-3,
        algorithmic_bytes=lambda r, c: 3 * r * c * 4,
    ),
    "lars_momentum": WorkloadSpec(
        name="lars_momentum", label="LARS momentum", category="optimizer",
        rows=4096, cols=65536, dtype=torch.float32, input_factory=make_lars_inputs, eps=1.0e-6,
        modeled_bytes_per_element=32.0, reread_bytes_per_element=12.0, staged_bytes_per_element=12,
        reductions_per_stage=(2,), atol=3.0e-3, rtol=3.0e-3,
        algorithmic_bytes=lambda r, c: 5 * r * c * 4,
    ),
    "rowwise_quant": WorkloadSpec(
        name="rowwise_quant", label="Row-wise int8 quantization", category="quantization",
        rows=4096, cols=65536, dtype=torch.float32, input_factory=make_quant_inputs, eps=0.0,
        modeled_bytes_per_element=9.0, reread_bytes_per_element=4.0, staged_bytes_per_element=4,
        reductions_per_stage=(1,), atol=1.0e-6, rtol=1.0e-6,
        algorithmic_bytes=lambda r, c: r * c * 5 + r * 4,
    ),
}


def algorithmic_bytes(name: str, rows: int, cols: int) -> int:
    return int(WORKLOADS[name].algorithmic_bytes(rows, cols))
