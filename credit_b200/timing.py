"""CUDA-event timing shared by the evaluation pipeline and bench.py.

One helper for every "time this callable on the device" need: warm-up calls, then
`trials` batches of `iterations` back-to-back calls, each batch bracketed by a pair of
events recorded on the stream the calls are launched on. The reference times its
in-process launchers the same way (`dsmem_eval/runner.py:166-182`) and its executables
with `time_kernel` (`src/workloads/layernorm_backward.cu:150-175`).
"""
from __future__ import annotations

from typing import Callable, Sequence

import numpy as np


def event_timed_batches(fn: Callable[[], None], warmup: int, iterations: int, trials: int = 1,
                        stream=None) -> list[float]:
    """Milliseconds per call for each of `trials` batches. `stream` defaults to torch's current
    stream, which must be the one `fn` launches on (an event only sees its own stream)."""
    import torch

    stream = stream if stream is not None else torch.cuda.current_stream()
    for _ in range(max(warmup, 0)):
        fn()
    stream.synchronize()
    per_call = []
    for _ in range(trials):
        first = torch.cuda.Event(enable_timing=True)
        last = torch.cuda.Event(enable_timing=True)
        first.record(stream)
        for _ in range(iterations):
            fn()
        last.record(stream)
        last.synchronize()
        per_call.append(first.elapsed_time(last) / iterations)
    return per_call


def quantiles(samples: Sequence[float], fractions: Sequence[float] = (0.2, 0.5, 0.8)) -> list[float]:
    """Linear-interpolation quantiles of the finite samples; NaN for each when none is finite."""
    values = np.asarray([float(v) for v in samples], dtype=np.float64)
    values = values[np.isfinite(values)]
    if values.size == 0:
        return [float("nan")] * len(fractions)
    return [float(q) for q in np.quantile(values, list(fractions))]
