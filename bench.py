"""Benchmark of the wide-row hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (config.workload): row-wise sum / max / argmax of an fp32 matrix
X [512, 1048576] ~ N(0,1) with one planted +10 per row, generated on the device from a
fixed seed (synthetic data). One step = one pass of the kernel over one such matrix.
With N ranks (one process per GPU, launched by torchrun) every rank reduces its own 512
rows: rows are independent, there is no collective on the data path, so scaling is weak
and `value` is N * 512 * K / (slowest rank's time).

The JSON line also carries
  e2e        the same metric through the host-buffer C-ABI call
             (credit_row_reduce_host): pinned host input -> device -> results in
             host memory, copies inside the timed region;
  roofline   algorithmic bytes per launch / mean launch time (CUDA events on the
             launching stream) against the measured HBM copy ceiling; `traffic` is the
             DRAM traffic of one launch from the ncu capture recorded in
             profiles/ncu_traffic.json;
  cpu_baseline  the CPU oracle (torch, all host threads) on a bounded row sample;
  others     (N = 1) every other target shape as a measurement of its own: RMSNorm
             forward, LayerNorm forward, LayerNorm backward with dgamma/dbeta and the
             fused FFN, each with device time, roofline, cpu_baseline, e2e through its
             host-buffer entry point and the clocks sampled during its own timed region;
  strong     (N > 1) every target shape split into row blocks over the ranks
             (rows / N per GPU) beside the same shape run whole on every GPU, and the
             check of the all-reduced dgamma/dbeta against an fp64 computation.

--impl reference times the CPU oracle alone (rank 0 only under torchrun).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

ROWS, COLS = 512, 1048576
WORKLOAD = "row_reduce fp32 [512, 1048576] -> sum, max, argmax(int64)"
METRIC = "row_reduce_rows_per_s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
FFN_SHAPE = (2048, 4096, 16384)   # m, d, h
# (key, workload, rows, cols): the target shapes of the staged row kernels
ROW_CASES = [
    ("rmsnorm_forward", "rmsnorm_forward", 1024, 32768),
    ("layernorm_forward", "layernorm_forward", 4096, 131072),
    ("layernorm_backward_stats", "layernorm_backward_stats", 8192, 65536),
    # the reference's own workload (statistics recomputed, dx only) at the largest shape of its sweep
    ("layernorm_backward_reference_form", "layernorm_backward", 2048, 65536),
]
E2E_KEYS = ("rmsnorm_forward", "layernorm_forward", "layernorm_backward_stats")   # workloads with a host-buffer entry point
OTHER_ITERS = 50
BURST_IDLE_S = 1.0     # idle time before a burst measurement
SUSTAINED_S = 1.5     # length of the back-to-back run reported beside each burst figure


def measured_peaks() -> dict:
    """Roofline denominators: the driver-measured file if present, else the fallbacks."""
    peaks = {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
             "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            peaks.update({k: float(raw[k]) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained") if k in raw})
            peaks["source"] = "measured"
        except Exception:
            pass
    return peaks


def ncu_traffic(key: str) -> int | None:
    """dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch, scaled from the
    capture recorded beside the ncu summaries (traffic of these kernels is per row)."""
    path = ROOT / "profiles" / "ncu_traffic.json"
    try:
        entry = json.loads(path.read_text())[key]
        scale = entry["rows_full"] / entry["rows_captured"]
        return int((entry["dram_bytes_read"] + entry["dram_bytes_write"]) * scale)
    except Exception:
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, uuid: str | None = None, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples: list[tuple[float, int, int]] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            try:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid) if uuid else None
            except Exception:
                self._handle = None
            if self._handle is None:
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _loop(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                self.samples.append((time.perf_counter(), int(mhz), int(reasons)))
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, windows: list[tuple[float, float]]) -> dict:
        inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in windows)]
        chosen = inside if len(inside) >= 2 else self.samples
        if not chosen:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        bits = 0
        for _, _, r in chosen:
            bits |= r
        return {
            "sm_mhz": statistics.median(m for _, m, _ in chosen),
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(name for bit, name in self.REASONS.items() if bits & bit),
            "samples": len(chosen),
            "in_window": len(inside) >= 2,
        }


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every logical CPU of the box at any N."""
    import torch
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def time_cpu(fn, budget_s: float) -> tuple[float, int]:
    """Median seconds per call over at least 3 calls, stopping after `budget_s`."""
    fn()  # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 40):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return statistics.median(times), len(times)


def cpu_baseline(max_seconds: float = 10.0) -> dict:
    """The CPU oracle on a bounded sample of the headline workload: 32 of the 512 rows per call."""
    from credit_b200 import workloads as W
    from oracle import reference_ops as O

    cores = use_all_host_threads()
    sample_rows = 32
    (x,) = W.make_row_reduce_inputs(sample_rows, COLS, "cpu")
    med, n = time_cpu(lambda: O.row_reduce(x), max_seconds)
    return {
        "value": sample_rows / med, "unit": "rows/s", "cores": cores, "kind": "port",
        "sample": f"{sample_rows} of {ROWS} rows x {COLS} cols per call, median of {n} calls "
                  f"(torch CPU sum/amax/argmax, {os.cpu_count()} logical CPUs on the box)",
    }


def cpu_baseline_for(key: str, budget_s: float = 4.0) -> dict:
    """The CPU oracle of one of the other target shapes on a bounded block of rows (rows are
    independent; LayerNorm backward's column sums are taken over the block)."""
    import torch
    from credit_b200 import workloads as W
    from oracle import reference_ops as O

    cores = use_all_host_threads()
    if key == "ffn_forward":
        m, d, h = FFN_SHAPE
        sample = 64
        x, w1, w2, gamma = W.make_ffn_inputs(sample, d, "cpu", hidden=h)
        w1f, w2f = w1.float(), w2.float()   # a CPU implementation keeps its weights in its compute type
        med, n = time_cpu(lambda: O.ffn_forward(x, w1f, w2f, gamma), budget_s)
        what, total = "torch CPU fp32 matmul + erf GELU + RMSNorm", m
    else:
        name, rows, cols = next((w, r, c) for k, w, r, c in ROW_CASES if k == key)
        sample = {"rmsnorm_forward": 128, "layernorm_forward": 32, "layernorm_backward_stats": 64,
                  "layernorm_backward_reference_form": 64}[key]
        ins = W.WORKLOADS[name].input_factory(sample, cols, "cpu")
        fn = {"rmsnorm_forward": O.rmsnorm_forward, "layernorm_forward": O.layernorm_forward,
              "layernorm_backward_stats": O.layernorm_backward_stats,
              "layernorm_backward_reference_form": O.layernorm_backward}[key]
        med, n = time_cpu(lambda: fn(*ins), budget_s)
        what, total = "torch CPU, fp32 arithmetic", rows
    return {"value": sample / med, "unit": "rows/s", "cores": cores, "kind": "port",
            "sample": f"{sample} of {total} rows per call, median of {n} calls ({what})"}


def run_reference_arm(args) -> None:
    """Times the CPU implementation of the path (the oracle port) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from credit_b200 import workloads as W
    from oracle import reference_ops as O

    cores = use_all_host_threads()
    sample_rows = 16
    (x,) = W.make_row_reduce_inputs(sample_rows, COLS, "cpu")
    for _ in range(max(1, args.warmup)):
        O.row_reduce(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.row_reduce(x)
    elapsed = time.perf_counter() - t0
    value = sample_rows * args.steps / elapsed
    sample = (f"each step = {sample_rows} of {ROWS} rows x {COLS} cols (torch CPU sum/amax/argmax, "
              f"{cores} threads)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * elapsed / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": ROWS, "cols": COLS,
                   "note": "CPU arm: bounded row sample per step, all host threads at every N"},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit_result(line)


# ---------------------------------------------------------------------------------------------
# device-side measurements
# ---------------------------------------------------------------------------------------------
class RowCase:
    """One staged row workload at a given shape: rotating input sets (so that a shape that fits
    the L2 is not timed out of it), outputs, workspace, and the call."""

    def __init__(self, name: str, rows: int, cols: int, dev, seed: int = 0):
        import torch
        from credit_b200 import launchers as L
        from credit_b200 import workloads as W

        self.name, self.rows, self.cols = name, rows, cols
        spec = W.WORKLOADS[name]
        self.dtype = spec.dtype
        self.bytes = W.algorithmic_bytes(name, rows, cols)
        # about 1 GiB (8x the 126 MB L2) of other traffic between two uses of the same buffers,
        # in at most 8 sets
        self.nsets = max(1, min(8, -(-(1 << 30) // max(self.bytes, 1))))
        self.sets = []
        for s in range(self.nsets):
            ins = spec.input_factory(rows, cols, dev, seed=seed + s)
            self.sets.append((ins, L.allocate_outputs(name, ins)))
        self.kw = {}
        if name == "layernorm_backward_stats":
            need = L.layernorm_backward_stats_workspace_bytes(rows, cols, spec.dtype)
            self.kw["workspace"] = torch.empty(need, dtype=torch.uint8, device=dev)
        self._i = 0
        self._launcher = L.NATIVE_LAUNCHERS[name]

    def call(self):
        ins, outs = self.sets[self._i % self.nsets]
        self._i += 1
        self._launcher(ins, outs, 0, None, **self.kw)

    def l2_note(self) -> str:
        return (f"{self.nsets} rotating buffer sets" if self.nsets > 1
                else "inputs of one launch are larger than the 126 MB L2")


def idle_before_burst() -> None:
    """A burst figure is a kernel timed from an idle GPU: the previous workload's sustained loop leaves
    the board at its power limit for a few hundred milliseconds (the `clocks` block of each figure
    shows which state it was measured in)."""
    import torch
    torch.cuda.synchronize()
    time.sleep(BURST_IDLE_S)


def timed_ms(fn, iters: int, warmup: int = 3, min_region_ms: float = 0.0):
    """ms per call (CUDA events on the current stream), the wall-clock window of the region and
    the iterations timed. With `min_region_ms` the iteration count grows until the timed region
    lasts that long, so that the clock sampler sees it (estimated from the warm-up calls)."""
    from credit_b200.timing import event_timed_batches
    import torch
    if warmup > 0:
        (est,) = event_timed_batches(fn, 0, warmup, 1)
        if min_region_ms > 0 and est > 0:
            iters = max(iters, int(min_region_ms / est) + 1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    (ms,) = event_timed_batches(fn, 0, iters, 1)
    torch.cuda.synchronize()
    return ms, (t0, time.perf_counter()), iters


def pinned_like(t):
    import torch
    return torch.empty(t.shape, dtype=t.dtype, pin_memory=True)


def e2e_row_case(key: str, case: RowCase, dev, steps: int = 5) -> dict:
    """The workload through its host-buffer entry point: pinned host inputs, results back in host
    memory, every copy inside the timed region (wall clock: the call returns when the results are
    in host memory)."""
    import torch
    from credit_b200 import host as H

    ins, outs = case.sets[0]
    host_in = [pinned_like(t).copy_(t) for t in ins]
    host_out = [pinned_like(t) for t in outs]
    scratch = torch.empty(max(H.scratch_bytes(case.name, case.rows, case.cols, case.dtype), 1 << 30),
                          dtype=torch.uint8, device=dev)
    call = {
        "rmsnorm_forward": lambda: H.rmsnorm_forward(host_in[0], host_in[1], host_out[0], scratch),
        "layernorm_forward": lambda: H.layernorm_forward(*host_in, *host_out, scratch),
        "layernorm_backward_stats": lambda: H.layernorm_backward_stats(*host_in, *host_out, scratch),
    }[key]
    call()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        call()
    elapsed = time.perf_counter() - t0
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    return {"value": case.rows * steps / elapsed, "unit": "rows/s", "steps": steps, "ms_per_step": 1e3 * elapsed / steps,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "path": f"credit_{case.name}_host (pinned host buffers, copies inside the timed region)"}


def measure_row_case(key: str, name: str, rows: int, cols: int, dev, sampler, peaks, with_e2e: bool) -> dict:
    import torch
    from credit_b200 import _native as N

    case = RowCase(name, rows, cols, dev)
    wl = {"rmsnorm_forward": N.WL_RMSNORM_FORWARD, "layernorm_forward": N.WL_LAYERNORM_FORWARD,
          "layernorm_backward_stats": N.WL_LAYERNORM_BACKWARD_STATS, "layernorm_backward": N.WL_LAYERNORM_BACKWARD}[name]
    plan = N.plan(wl, rows, cols, N.BF16 if case.dtype == torch.bfloat16 else N.F32)
    idle_before_burst()
    ms, window, iters = timed_ms(case.call, OTHER_ITERS, min_region_ms=120.0)
    achieved = case.bytes / ms / 1e6
    entry = {
        "shape": [rows, cols], "dtype": str(case.dtype).replace("torch.", ""), "ms": round(ms, 4),
        "iters": iters, "rows_per_s": round(rows / ms * 1e3, 1), "gbps": round(achieved, 1),
        "config": {"cluster_size": plan.cluster_size, "threads": plan.threads, "stages": plan.stages,
                   "grid_ctas": plan.grid_ctas, "choice": "automatic (the planner's model)", "l2": case.l2_note()},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth",
                     "algorithmic_bytes_per_launch": case.bytes, "traffic": ncu_traffic(key),
                     "frac_of_nominal_8TBs": achieved / 8000.0},
        "gpu_launches": iters * plan.kernel_launches,
        "clocks": sampler.summary([window]),
    }
    # The same call back to back for SUSTAINED_S seconds: these kernels draw the board's 1000 W limit
    # after about 0.1 s of continuous streaming, the SM clock settles near 1.7 GHz, and a kernel whose
    # output warps are close to their issue limit slows with it (a pure stream does not).
    s_ms, s_window, s_iters = timed_ms(case.call, max(OTHER_ITERS, int(SUSTAINED_S * 1e3 / ms) + 1), warmup=0)
    s_achieved = case.bytes / s_ms / 1e6
    entry["sustained"] = {"ms": round(s_ms, 4), "iters": s_iters, "seconds": round(s_window[1] - s_window[0], 2),
                          "gbps": round(s_achieved, 1), "frac": s_achieved / peaks["hbm_gbs"],
                          "clocks": sampler.summary([s_window])}
    entry["gpu_launches"] += s_iters * plan.kernel_launches
    if with_e2e:
        try:
            entry["e2e"] = e2e_row_case(key, case, dev)
        except Exception as exc:  # report, do not hide
            entry["e2e"] = {"error": str(exc)[:200]}
    del case
    torch.cuda.empty_cache()
    return entry


def measure_ffn(dev, sampler, peaks, m: int | None = None, with_e2e: bool = True, sustained_s: float = 2.0) -> dict:
    """The fused FFN: a burst of 50 calls against the measured burst bf16 peak, then a loop of at
    least `sustained_s` seconds against the sustained one (the GPU runs into its power cap)."""
    import torch
    from credit_b200 import host as H
    from credit_b200 import launchers as L
    from credit_b200 import workloads as W

    full_m, d, h = FFN_SHAPE
    m = full_m if m is None else m
    x, w1, w2, gamma = W.make_ffn_inputs(m, d, dev, hidden=h)
    w1p, w2p = L.pack_ffn_weight(w1), L.pack_ffn_weight(w2)
    del w1, w2
    y = torch.empty_like(x)
    ws = torch.empty(L.ffn_workspace_bytes(m, d, h), dtype=torch.uint8, device=dev)

    def call():
        L.launch_ffn_forward((x, w1p, w2p, gamma), (y,), workspace=ws)

    flops = W.ffn_flops(m, d, h)
    ms, window, _ = timed_ms(call, OTHER_ITERS)
    tflops = flops / ms / 1e9
    entry = {
        "shape": [m, d, h], "dtype": "bfloat16", "ms": round(ms, 4), "iters": OTHER_ITERS,
        "tflops": round(tflops, 1), "rows_per_s": round(m / ms * 1e3, 1),
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": tflops / peaks["bf16_tflops"], "peak_source": f"{peaks['source']} cuBLAS bf16, burst",
                     "flops_per_call": flops, "traffic": ncu_traffic("ffn_forward"),
                     "frac_of_nominal_2250": tflops / 2250.0},
        "gpu_launches": 2 * OTHER_ITERS,
        "clocks": sampler.summary([window]),
    }
    if sustained_s > 0:
        n = max(OTHER_ITERS, int(sustained_s / (ms * 1e-3)) + 1)
        ms_s, window_s, _ = timed_ms(call, n, warmup=0)
        tf_s = flops / ms_s / 1e9
        entry["sustained"] = {"ms": round(ms_s, 4), "iters": n, "seconds": round(ms_s * n * 1e-3, 2),
                              "tflops": round(tf_s, 1), "peak": peaks["bf16_tflops_sustained"],
                              "frac": tf_s / peaks["bf16_tflops_sustained"],
                              "clocks": sampler.summary([window_s])}
    if with_e2e:
        try:
            hx, hy = pinned_like(x).copy_(x), pinned_like(y)
            scratch = torch.empty(H.scratch_bytes("ffn_forward", m, d, hidden=h), dtype=torch.uint8, device=dev)
            H.ffn_forward(hx, w1p, w2p, gamma, hy, scratch)
            steps = 10
            t0 = time.perf_counter()
            for _ in range(steps):
                H.ffn_forward(hx, w1p, w2p, gamma, hy, scratch)
            elapsed = time.perf_counter() - t0
            nbytes = hx.numel() * 2
            entry["e2e"] = {"value": m * steps / elapsed, "unit": "rows/s", "steps": steps,
                            "ms_per_step": 1e3 * elapsed / steps, "h2d_bytes_per_step": nbytes,
                            "d2h_bytes_per_step": nbytes,
                            "path": "credit_ffn_forward_host (activations in pinned host memory, weights resident)"}
        except Exception as exc:
            entry["e2e"] = {"error": str(exc)[:200]}
    del x, y, w1p, w2p, ws
    torch.cuda.empty_cache()
    return entry


def others_single_gpu(dev, sampler, peaks) -> dict:
    out = {}
    # the FFN first (tensor-bound, power-capped), before the memory-bound kernels have heated the GPU
    for key, fn in [("ffn_forward", lambda: measure_ffn(dev, sampler, peaks))] + [
            (key, (lambda k=key, n=name, r=rows, c=cols: measure_row_case(k, n, r, c, dev, sampler, peaks, k in E2E_KEYS)))
            for key, name, rows, cols in ROW_CASES]:
        try:
            out[key] = fn()
        except Exception as exc:  # report, do not hide
            out[key] = {"error": str(exc)[:300]}
    for key in out:
        if "error" not in out[key]:
            try:
                out[key]["cpu_baseline"] = cpu_baseline_for(key)
            except Exception as exc:
                out[key]["cpu_baseline"] = {"error": str(exc)[:200]}
    return out


def max_over_ranks(value: float, dev) -> float:
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], device=dev, dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def multi_gpu_blocks(dev, rank: int, world: int) -> dict:
    """N > 1. (1) The path's only collective: LayerNorm backward on each rank's rows followed by
    the all-reduce of dgamma/dbeta over NVLink, timed together on the device, and the all-reduced
    result checked against an fp64 computation of the same column sums. (2) Strong scaling: every
    target shape split into contiguous row blocks (rows / N per GPU) beside the same shape run
    whole on every GPU (weak), device time, max over ranks."""
    import torch
    import torch.distributed as dist
    from credit_b200 import launchers as L
    from credit_b200 import sharding
    from credit_b200 import workloads as W

    out: dict = {}
    iters = 20

    def sharded_backward(rows_total: int, cols: int, split: bool, peer_group=None):
        r0, r1 = sharding.shard_rows(rows_total, world, rank) if split else (0, rows_total)
        rows = r1 - r0
        ins = W.make_layernorm_backward_stats_inputs(rows, cols, dev, seed=rank)
        dx = torch.empty_like(ins[0])
        both, _, _ = sharding.allocate_param_grads(cols, dev)
        ws = torch.empty(L.layernorm_backward_stats_workspace_bytes(rows, cols, ins[0].dtype),
                         dtype=torch.uint8, device=dev)

        def call():
            sharding.layernorm_backward_stats_sharded(ins, dx, both, workspace=ws, peer_group=peer_group)
        return ins, both, call

    def time_call(call):
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        dist.barrier()
        ms, _, _ = timed_ms(call, iters, warmup=0)
        return max_over_ranks(ms, dev)

    # ---- the collective, whole shape per GPU (weak), with the check of its result
    c_rows, c_cols = 8192, 65536
    ins, both, call = sharded_backward(c_rows, c_cols, split=False)
    weak_ms = time_call(call)
    x, dy, _, mean, rstd = ins
    want = torch.zeros((2, c_cols), dtype=torch.float64, device=dev)
    for r0 in range(0, c_rows, 512):       # fp64 column sums of this rank's rows, in row chunks
        xs, ds = x[r0:r0 + 512].double(), dy[r0:r0 + 512].double()
        xhat = (xs - mean[r0:r0 + 512, None].double()) * rstd[r0:r0 + 512, None].double()
        want[0] += (ds * xhat).sum(0)
        want[1] += ds.sum(0)
    dist.all_reduce(want)                  # fp64 sum over the ranks: independent of the fp32 path
    err = (both.double() - want).abs()
    tol = 1e-5 * want.abs() + 1e-5 * 4.0 * (world * c_rows) ** 0.5
    worst = float((err / tol).max().item())
    worst = max_over_ranks(worst, dev)
    out["collective_check"] = {"status": "ok" if worst <= 1.0 else "FAILED", "worst_error_over_tolerance": round(worst, 4),
                               "what": "all-reduced dgamma/dbeta of the last timed call vs fp64 column sums "
                                       "all-reduced in fp64; tolerance 1e-5 relative + 1e-5 * 4 * sqrt(total rows)"}
    if worst > 1.0:
        raise SystemExit(f"all-reduced dgamma/dbeta are wrong (error / tolerance = {worst})")
    # ---- the same step with the library's own all-reduce over peer memory (one kernel per rank, CUDA
    # IPC windows); every rank agrees at each stage before the next collective step is taken
    def all_ok(flag: bool, payload=None):
        gathered: list = [None] * world
        dist.all_gather_object(gathered, (bool(flag), payload))
        return all(g[0] for g in gathered), [g[1] for g in gathered]

    peer = {"status": "unavailable"}
    group = None
    try:
        try:
            group = sharding.PeerGroup(world, rank, c_cols, connect=False)
            created, note = True, ""
        except Exception as exc:
            created, note = False, str(exc)[:200]
        everyone, handles = all_ok(created, group.handle if created else None)
        if everyone:
            try:
                group.connect(handles)
                connected = True
            except Exception as exc:
                connected, note = False, str(exc)[:200]
            everyone, _ = all_ok(connected)
        if everyone:
            _, both_p, call_p = sharded_backward(c_rows, c_cols, split=False, peer_group=group)
            # same seeds as above: the fp64 column sums in `want` are the expected result here too
            peer_ms = time_call(call_p)
            perr = float(((both_p.double() - want).abs() / tol).max().item())
            # the collective alone, back to back on a scratch copy (values grow, timing does not care)
            scratch_both = both_p.clone()
            only_nccl = time_call(lambda: sharding.allreduce_param_grads(scratch_both))
            scratch_both.copy_(both_p)
            only_peer = time_call(lambda: group.allreduce(scratch_both))
            del scratch_both
            perr = max_over_ranks(perr, dev)
            status = max_over_ranks(float(group.status()), dev)
            peer = {"status": "ok" if perr <= 1.0 and status == 0 else "FAILED", "ms": round(peer_ms, 4),
                    "rows_per_s": round(world * c_rows / peer_ms * 1e3, 1), "worst_error_over_tolerance": round(perr, 4),
                    "against_nccl_ms": round(weak_ms, 4),
                    "allreduce_alone_us": {"nccl": round(only_nccl * 1e3, 1), "peer": round(only_peer * 1e3, 1)},
                    "what": "credit_layernorm_bwd_allreduce_peer: each rank publishes its [2, cols] vector in a "
                            "window its peers map, one flag per rank, sums in rank order (plain NVLink loads)"}
            del both_p, call_p
            # a wrong or timed-out peer all-reduce is reported, not fatal: the headline and the NCCL path
            # above do not depend on it
        else:
            peer = {"status": "unavailable", "why": note or "another rank could not create or map its window"}
    finally:
        torch.cuda.synchronize()
        dist.barrier()          # nobody closes a window a peer may still read
        if group is not None:
            group.close()
    out["peer_allreduce"] = peer
    del ins, both, call, want, err, tol, x, dy
    torch.cuda.empty_cache()
    ins, both, call = sharded_backward(c_rows, c_cols, split=True)
    strong_ms = time_call(call)
    del ins, both, call
    torch.cuda.empty_cache()
    out["layernorm_backward_stats_sharded"] = {
        "shape": [c_rows, c_cols], "dtype": "bfloat16",
        "allreduce": f"dgamma/dbeta, {2 * c_cols * 4} B fp32 over NCCL, in place, same stream",
        "weak": {"rows_per_gpu": c_rows, "ms": round(weak_ms, 4), "rows_per_s": round(world * c_rows / weak_ms * 1e3, 1)},
        "strong": {"rows_per_gpu": c_rows // world, "ms": round(strong_ms, 4),
                   "rows_per_s": round(c_rows / strong_ms * 1e3, 1),
                   "speedup_vs_whole_shape_on_one_gpu": round(weak_ms / strong_ms, 3),
                   "efficiency": round(weak_ms / strong_ms / world, 3)},
    }

    # ---- the workloads without any collective
    strong = {}
    cases = [("row_reduce", "row_reduce", ROWS, COLS)] + [c for c in ROW_CASES if c[0] != "layernorm_backward_stats"]
    for key, name, rows, cols in cases:
        try:
            r0, r1 = sharding.shard_rows(rows, world, rank)
            whole = RowCase(name, rows, cols, dev, seed=rank)
            weak = time_call(whole.call)
            del whole
            torch.cuda.empty_cache()
            part = RowCase(name, r1 - r0, cols, dev, seed=rank)
            strong_t = time_call(part.call)
            del part
            torch.cuda.empty_cache()
            strong[key] = {"shape": [rows, cols], "rows_per_gpu": r1 - r0, "weak_ms": round(weak, 4),
                           "weak_rows_per_s": round(world * rows / weak * 1e3, 1), "strong_ms": round(strong_t, 4),
                           "strong_rows_per_s": round(rows / strong_t * 1e3, 1),
                           "speedup_vs_whole_shape_on_one_gpu": round(weak / strong_t, 3),
                           "efficiency": round(weak / strong_t / world, 3)}
        except Exception as exc:
            strong[key] = {"error": str(exc)[:200]}
    try:
        m, d, h = FFN_SHAPE
        r0, r1 = sharding.shard_rows(m // 128, world, rank)     # whole 128-row blocks per rank
        peaks = measured_peaks()

        class _NoClocks:
            def summary(self, windows):
                return {}
        whole = measure_ffn(dev, _NoClocks(), peaks, m=m, with_e2e=False, sustained_s=0.0)
        weak = max_over_ranks(whole["ms"], dev)
        part_rows = max(128, (r1 - r0) * 128)
        part = measure_ffn(dev, _NoClocks(), peaks, m=part_rows, with_e2e=False, sustained_s=0.0)
        strong_t = max_over_ranks(part["ms"], dev)
        strong["ffn_forward"] = {"shape": list(FFN_SHAPE), "rows_per_gpu": part_rows, "weak_ms": round(weak, 4),
                                 "strong_ms": round(strong_t, 4), "strong_rows_per_s": round(m / strong_t * 1e3, 1),
                                 "speedup_vs_whole_shape_on_one_gpu": round(weak / strong_t, 3),
                                 "efficiency": round(weak / strong_t / world, 3),
                                 "note": "weights replicated: every rank still streams W1 and W2 in full"}
    except Exception as exc:
        strong["ffn_forward"] = {"error": str(exc)[:200]}
    out["strong"] = strong
    return out


_RESULT_FD = None


def keep_stdout_for_the_result() -> None:
    """Libraries print to stdout too (NCCL announces its version there on the first collective).
    Everything written to fd 1 from here on goes to stderr; the JSON line is written to the saved
    descriptor, so stdout carries exactly that one line."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit_result(line: dict) -> None:
    text = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-others", action="store_true", help="headline workload only")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup
    keep_stdout_for_the_result()

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from credit_b200 import _native as N
    from credit_b200 import host as H
    from credit_b200 import launchers as L
    from credit_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    N.load()

    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        uuid = None
    sampler = ClockSampler(local_rank, uuid)
    sampler.start()
    peaks = measured_peaks()

    # ---- inputs resident in HBM (2 GiB per launch, 17x the 126 MB L2)
    (x,) = W.make_row_reduce_inputs(ROWS, COLS, dev, seed=rank)
    outs = L.allocate_outputs("row_reduce", (x,))
    plan = N.plan(N.WL_ROW_REDUCE, ROWS, COLS, N.F32)
    stream = torch.cuda.current_stream()

    def step():
        L.launch_row_reduce((x,), outs)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_w0 = time.perf_counter()
    start.record(stream)
    for _ in range(args.steps):
        step()
    stop.record(stream)
    stop.synchronize()
    torch.cuda.synchronize()
    t_w1 = time.perf_counter()
    elapsed_ms = start.elapsed_time(stop)
    if N.device_status() != 0:
        raise SystemExit("a kernel reported a timeout or bad geometry")
    max_ms = max_over_ranks(elapsed_ms, dev)
    value = world * ROWS * args.steps / (max_ms * 1e-3)

    # sanity on the result of the timed launches: the planted maximum
    assert bool((outs[1] == 10.0).all()), "row maxima are wrong"

    # ---- end to end through the host-buffer entry point
    e2e_steps = max(3, min(args.steps, 20))
    x_host = torch.empty((ROWS, COLS), dtype=torch.float32, pin_memory=True)
    x_host.copy_(x)
    h_sum = torch.empty(ROWS, dtype=torch.float32, pin_memory=True)
    h_max = torch.empty(ROWS, dtype=torch.float32, pin_memory=True)
    h_arg = torch.empty(ROWS, dtype=torch.int64, pin_memory=True)
    del x
    torch.cuda.empty_cache()
    scratch = torch.empty(max(H.scratch_bytes("row_reduce", ROWS, COLS), 512 << 20), dtype=torch.uint8, device=dev)

    def e2e_step():
        H.row_reduce(x_host, h_sum, h_max, h_arg, scratch)

    e2e_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t_e0 = time.perf_counter()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e_stop.record(stream)
    e_stop.synchronize()
    t_e1 = time.perf_counter()
    # the call returns when the results are in host memory: wall time is the honest clock
    e2e_ms = max_over_ranks(max((t_e1 - t_e0) * 1e3, e_start.elapsed_time(e_stop)), dev)
    e2e_value = world * ROWS * e2e_steps / (e2e_ms * 1e-3)
    assert bool((h_max == 10.0).all()), "host results are wrong"
    # blocks per call: the library halves the block until two sets fit the scratch it was given
    block_rows, row_bytes = ROWS, COLS * 4 + 16
    while block_rows > 1 and 2 * block_rows * row_bytes > scratch.numel():
        block_rows = (block_rows + 1) // 2
    e2e_launches = e2e_steps * -(-ROWS // block_rows)
    del scratch, x_host
    torch.cuda.empty_cache()
    headline_clocks = sampler.summary([(t_w0, t_w1), (t_e0, t_e1)])

    multi = {}
    if world > 1 and not args.no_others:
        multi = multi_gpu_blocks(dev, rank, world)

    if rank == 0:
        ms_per_launch = elapsed_ms / args.steps
        alg_bytes = W.algorithmic_bytes("row_reduce", ROWS, COLS)
        achieved = alg_bytes / (ms_per_launch * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": max_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {
                "workload": WORKLOAD, "rows_per_gpu": ROWS, "cols": COLS,
                "cluster_size": plan.cluster_size, "load_path": "tma" if plan.load_path == N.LOAD_TMA else "ldg",
                "threads": plan.threads, "grid_ctas": plan.grid_ctas,
                "l2": "input (2 GiB per launch) is 17x larger than the 126 MB L2; no flush needed",
                "timing": "CUDA events on the launching stream, max over ranks",
            },
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth "
                "(a read-only kernel can exceed a copy)",
                "algorithmic_bytes_per_launch": alg_bytes,
                "traffic": ncu_traffic("row_reduce"),
                "frac_of_nominal_8TBs": achieved / 8000.0,
            },
            "e2e": {
                "value": e2e_value, "unit": "rows/s", "steps": e2e_steps,
                "h2d_bytes_per_step": ROWS * COLS * 4, "d2h_bytes_per_step": ROWS * 16,
                "path": "credit_row_reduce_host (pinned host buffers, copies inside the timed region)",
            },
            "gpu_launches": args.steps * plan.kernel_launches,
            "gpu_launches_e2e": e2e_launches,
            "clocks": headline_clocks,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline()
            if not args.no_others:
                line["others"] = others_single_gpu(dev, sampler, peaks)
        line.update(multi)
        sampler.stop()
        emit_result(line)
    else:
        sampler.stop()

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
