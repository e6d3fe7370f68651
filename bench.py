"""Benchmark of the wide-row hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (config.workload): row-wise sum / max / argmax of an fp32 matrix
X [512, 1048576] ~ N(0,1) with one planted +10 per row, generated on the device
from a fixed seed (synthetic data). One step = one pass of the kernel over
one such matrix. With N ranks (one process per GPU, launched by torchrun) every
rank reduces its own 512 rows: rows are independent, there is no collective on the
data path, so scaling is weak and `value` is N * 512 * K / (slowest rank's time).

The JSON line also carries
  e2e        the same metric through the host-buffer C-ABI call
             (credit_row_reduce_host): pinned host input -> device -> results in
             host memory, copies inside the timed region;
  roofline   algorithmic bytes per launch / mean launch time (CUDA events on the
             launching stream) against the measured HBM copy ceiling;
  cpu_baseline  the CPU oracle (torch, all host threads) on a bounded row sample;
  others     device-timed GB/s of the other wide-row workloads at their headline
             shapes (N = 1 only), for context.

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
# dram__bytes_read.sum + dram__bytes_write.sum per full-size launch: the ncu capture summarised in
# profiles/row_reduce_ncu_full.md was taken on 128 rows of the same width (536 888 064 B read +
# 5 983 232 B written) and is scaled by 4 to the 512 rows of a launch (traffic is per row).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 4 * (536_888_064 + 5_983_232)


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, uuid: str | None = None, period_s: float = 0.02):
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
        }


def cpu_baseline(max_seconds: float = 12.0) -> dict:
    """The CPU oracle on a bounded sample of the workload: 32 of the 512 rows per call."""
    import torch
    from credit_b200 import workloads as W
    from oracle import reference_ops as O

    sample_rows = 32
    (x,) = W.make_row_reduce_inputs(sample_rows, COLS, "cpu")
    O.row_reduce(x)  # warm-up
    times = []
    t_end = time.perf_counter() + max_seconds
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 40):
        t0 = time.perf_counter()
        O.row_reduce(x)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {
        "value": sample_rows / med,
        "unit": "rows/s",
        "cores": torch.get_num_threads(),
        "kind": "port",
        "sample": f"{sample_rows} of {ROWS} rows x {COLS} cols per call, median of {len(times)} calls "
                  f"(torch CPU sum/amax/argmax, {os.cpu_count()} logical CPUs on the box)",
    }


def run_reference_arm(args) -> None:
    """Times the CPU implementation of the path (the oracle port) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from credit_b200 import workloads as W
    from oracle import reference_ops as O

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
              f"{torch.get_num_threads()} threads)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * elapsed / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": ROWS, "cols": COLS,
                   "note": "CPU arm: bounded row sample per step"},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit_result(line)


def time_other_workloads(torch, dev) -> dict:
    """Device-timed GB/s of the other headline shapes (context for the roofline)."""
    from credit_b200 import launchers as L
    from credit_b200 import workloads as W

    out = {}

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        b.synchronize()
        return a.elapsed_time(b) / iters

    # the fused FFN (tensor-bound, power-capped): TFLOP/s against the measured dense bf16 peak; timed
    # first, before the memory-bound kernels have heated the GPU
    try:
        m, d, h = 2048, 4096, 16384
        x, w1, w2, gamma = W.make_ffn_inputs(m, d, dev, hidden=h)
        w1p, w2p = L.pack_ffn_weight(w1), L.pack_ffn_weight(w2)
        del w1, w2
        y = torch.empty_like(x)
        ws = torch.empty(L.ffn_workspace_bytes(m, d, h), dtype=torch.uint8, device=dev)
        ms = timed(lambda: L.launch_ffn_forward((x, w1p, w2p, gamma), (y,), workspace=ws), 10)
        tflops = W.ffn_flops(m, d, h) / ms / 1e9
        entry = {"shape": [m, d, h], "dtype": "bfloat16", "ms": round(ms, 4), "tflops": round(tflops, 1),
                 "rows_per_s": round(m / ms * 1e3, 1)}
        peaks = ROOT / "MEASURED_PEAKS.json"
        if peaks.exists():
            burst = json.loads(peaks.read_text()).get("bf16_tflops")
            if burst:
                entry["frac_of_measured_bf16_burst"] = round(tflops / float(burst), 3)
        out["ffn_forward"] = entry
        del x, w1p, w2p, y, ws
        torch.cuda.empty_cache()
    except Exception as exc:
        out["ffn_forward"] = {"error": str(exc)[:200]}
    # (key, workload, rows, cols, iterations, launch options; None = the planner's own choice)
    cases = [
        ("rmsnorm_forward", "rmsnorm_forward", 1024, 32768, 20, None),
        ("layernorm_forward", "layernorm_forward", 4096, 131072, 8, None),
        # the measured-best configuration of the cluster-size sweep, which the planner's model
        # ranks 3 % behind its own pick (P = 8, 512 threads)
        ("layernorm_forward_p16_256", "layernorm_forward", 4096, 131072, 8,
         {"cluster_size": 16, "threads": 256, "stages": 3}),
        ("layernorm_backward_stats", "layernorm_backward_stats", 8192, 65536, 6, None),
    ]
    for key, name, rows, cols, iters, config in cases:
        try:
            spec = W.WORKLOADS[name]
            sets = []
            nsets = 4 if name == "rmsnorm_forward" else 1   # rotate buffers where one set fits in L2
            for s in range(nsets):
                ins = spec.input_factory(rows, cols, dev, seed=s)
                sets.append((ins, L.allocate_outputs(name, ins)))
            kw = {}
            if name == "layernorm_backward_stats":
                need = L.layernorm_backward_stats_workspace_bytes(rows, cols, spec.dtype)
                kw["workspace"] = torch.empty(need, dtype=torch.uint8, device=dev)
            state = {"i": 0}

            opts = dict(config) if config else None
            cluster_size = opts.pop("cluster_size", 0) if opts else 0

            def call():
                ins, outs = sets[state["i"] % nsets]
                state["i"] += 1
                L.NATIVE_LAUNCHERS[name](ins, outs, cluster_size, opts, **kw)

            ms = timed(call, iters)
            nbytes = W.algorithmic_bytes(name, rows, cols)
            out[key] = {"shape": [rows, cols], "dtype": str(spec.dtype).replace("torch.", ""),
                        "ms": round(ms, 4), "gbps": round(nbytes / ms / 1e6, 1),
                        "rows_per_s": round(rows / ms * 1e3, 1),
                        "config": config if config else "automatic"}
            del sets, kw
            torch.cuda.empty_cache()
        except Exception as exc:  # report, do not hide
            out[key] = {"error": str(exc)[:200]}
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
    ap.add_argument("--no-others", action="store_true", help="skip the context workloads")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup
    keep_stdout_for_the_result()

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from credit_b200 import _native as N
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

    # ---- inputs resident in HBM (4x the 126 MB L2 per launch, 2 GiB per matrix)
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
    t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_ms = float(t.item())
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
    lib = N.load()
    scratch_bytes = max(lib.credit_row_reduce_host_scratch_bytes(ROWS, COLS), 512 << 20)
    scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=dev)

    def e2e_step():
        N.check(lib.credit_row_reduce_host(x_host.data_ptr(), h_sum.data_ptr(), h_max.data_ptr(),
                                           h_arg.data_ptr(), ROWS, COLS, None, scratch.data_ptr(),
                                           scratch.numel(), stream.cuda_stream))

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
    e2e_ms = max((t_e1 - t_e0) * 1e3, e_start.elapsed_time(e_stop))
    te = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = world * ROWS * e2e_steps / (float(te.item()) * 1e-3)
    assert bool((h_max == 10.0).all()), "host results are wrong"
    # same block size as the library derives from the scratch it was given
    out_bytes = 2 * (-(-ROWS * 4 // 256) * 256) + (-(-ROWS * 8 // 256) * 256)
    block_rows = min(ROWS, (((scratch.numel() - out_bytes) // 2) // 256 * 256) // (COLS * 4))
    e2e_launches = e2e_steps * -(-ROWS // block_rows)
    del scratch

    # ---- the path's only collective (N > 1): LayerNorm backward on this rank's rows,
    # then the all-reduce of dgamma/dbeta over NVLink, timed together on the device
    collective_result = {}
    if world > 1 and not args.no_others:
        from credit_b200 import sharding
        c_rows, c_cols = 8192, 65536
        ins = W.make_layernorm_backward_stats_inputs(c_rows, c_cols, dev, seed=rank)
        dx = torch.empty_like(ins[0])
        both, _, _ = sharding.allocate_param_grads(c_cols, dev)
        ws = torch.empty(L.layernorm_backward_stats_workspace_bytes(c_rows, c_cols, ins[0].dtype),
                         dtype=torch.uint8, device=dev)
        for _ in range(3):
            sharding.layernorm_backward_stats_sharded(ins, dx, both, workspace=ws)
        torch.cuda.synchronize()
        dist.barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c_iters = 6
        c0.record(stream)
        for _ in range(c_iters):
            sharding.layernorm_backward_stats_sharded(ins, dx, both, workspace=ws)
        c1.record(stream)
        c1.synchronize()
        tc = torch.tensor([c0.elapsed_time(c1) / c_iters], device=dev, dtype=torch.float64)
        dist.all_reduce(tc, op=dist.ReduceOp.MAX)
        collective_result["layernorm_backward_stats_sharded"] = {
            "shape_per_gpu": [c_rows, c_cols], "dtype": "bfloat16", "ms": round(float(tc.item()), 4),
            "rows_per_s": round(world * c_rows / float(tc.item()) * 1e3, 1),
            "allreduce": f"dgamma/dbeta, {2 * c_cols * 4} B fp32 over NCCL, in place, same stream",
        }
        del ins, dx, ws
        torch.cuda.empty_cache()

    sampler.stop()
    clocks = sampler.summary([(t_w0, t_w1), (t_e0, t_e1)])

    if rank == 0:
        peak, peak_kind = measured_peaks()
        ms_per_launch = elapsed_ms / args.steps
        alg_bytes = W.algorithmic_bytes("row_reduce", ROWS, COLS)
        achieved = alg_bytes / (ms_per_launch * 1e-3) / 1e9
        others = dict(collective_result)
        baseline = None
        if world == 1:
            baseline = cpu_baseline()
            if not args.no_others:
                others = time_other_workloads(torch, dev)
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
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth "
                "(a read-only kernel can exceed a copy)",
                "algorithmic_bytes_per_launch": alg_bytes,
                "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                "frac_of_nominal_8TBs": achieved / 8000.0,
            },
            "e2e": {
                "value": e2e_value, "unit": "rows/s", "steps": e2e_steps,
                "h2d_bytes_per_step": ROWS * COLS * 4, "d2h_bytes_per_step": ROWS * 16,
                "path": "credit_row_reduce_host (pinned host buffers, copies inside the timed region)",
            },
            "gpu_launches": args.steps * plan.kernel_launches,
            "gpu_launches_e2e": e2e_launches,
            "clocks": clocks,
        }
        if baseline is not None:
            line["cpu_baseline"] = baseline
        if others:
            line["others"] = others
        emit_result(line)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
