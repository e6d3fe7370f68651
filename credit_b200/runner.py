"""Evaluation pipeline: spawns the workload executables and the micro-benchmarks,
collects their `RESULT,` / `CONTROL,` lines, scores the cost models and writes a
result bundle.

Mirrors the native half of the reference pipeline (`dsmem_eval/runner.py`:
`RunConfig` :34-89, `run_checked` :96-117, `summarize` :143-151, `parse_cuda_output`
:258-277, `run_cuda_trials` :280-310, `run_control_trials` :313-347, `build_summary`
:444-620, `run_suite` :623-794) with the same CSV column names where the quantity
exists. The Triton / torch.compile half of the reference pipeline is a comparison
baseline and is not part of this project. Cluster sizes 1..16 are accepted, and the
summary adds what the B200 target asks for: the predicted fastest cluster size next
to the measured one, and roofline columns.
"""
from __future__ import annotations

import csv
import json
import math
import subprocess
import time
from collections import defaultdict
from dataclasses import asdict, dataclass, fields, replace
from pathlib import Path
from typing import Any, Iterable

from . import cost_model
from .report import write_report
from .timing import event_timed_batches, quantiles
from .profile import make_b200_calibration, make_device_profile, parse_primitive_output, profile_as_dict
from .workloads import WORKLOADS

PACKAGE_DIR = Path(__file__).resolve().parent
BIN_DIR = PACKAGE_DIR / "bin"
DEFAULT_N_VALUES = (4096, 8192, 16384, 32768, 65536)
DEFAULT_CLUSTER_SIZES = (1, 2, 4, 8, 16)   # 1: the same pipeline with one CTA per row
CLI_WORKLOADS = ("layernorm_backward", "rmsnorm_forward", "row_reduce", "layernorm_forward",
                 "layernorm_backward_stats", "weighted_var_backward", "pearson_backward",
                 "softmax_logits_backward", "lars_momentum", "rowwise_quant")
_WORKLOAD_IDS = {"rmsnorm_forward": 0, "row_reduce": 1, "layernorm_forward": 2, "layernorm_backward": 3,
                 "layernorm_backward_stats": 4, "weighted_var_backward": 5, "pearson_backward": 6,
                 "softmax_logits_backward": 7, "lars_momentum": 8, "rowwise_quant": 9}


@dataclass(frozen=True)
class RunConfig:
    """What a sweep runs. The field names are the keys of the reference's configuration dict
    (`dsmem_eval/runner.py:34-60`) so that saved configurations stay interchangeable; `rows`
    (0 = each workload's default) is an addition."""
    workloads: tuple[str, ...] = CLI_WORKLOADS
    n_values: tuple[int, ...] = DEFAULT_N_VALUES
    cluster_sizes: tuple[int, ...] = DEFAULT_CLUSTER_SIZES
    warmup: int = 20
    iterations: int = 100
    trials: int = 5
    quick: bool = False
    profile_only: bool = False
    rows: int = 0

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "RunConfig":
        """Builds a validated configuration from a plain dict; absent keys keep their defaults and
        every value is coerced to its field's type (lists become tuples of int or str)."""
        coerced: dict[str, Any] = {}
        for field in fields(cls):
            if field.name not in raw:
                continue
            value = raw[field.name]
            if isinstance(field.default, tuple):
                item = type(field.default[0])
                value = tuple(item(v) for v in value)
            else:
                value = type(field.default)(value)
            coerced[field.name] = value
        config = cls(**coerced)
        config.validate()
        return config

    def validate(self) -> None:
        problems = []
        strangers = [w for w in self.workloads if w not in CLI_WORKLOADS]
        if strangers:
            problems.append("unknown workloads: " + ", ".join(sorted(set(strangers))))
        if not (self.workloads or self.profile_only):
            problems.append("at least one workload is required")
        if not self.n_values or min(self.n_values) <= 0:
            problems.append("n_values must contain positive integers")
        if not self.cluster_sizes or not set(self.cluster_sizes) <= {1, 2, 4, 8, 16}:
            problems.append("cluster_sizes must be selected from 1, 2, 4, 8 and 16")
        if self.warmup <= 0 or self.iterations <= 0 or self.trials <= 0:
            problems.append("warmup, iterations, and trials must be positive")
        if self.rows < 0:
            problems.append("rows must not be negative")
        if problems:
            raise ValueError("; ".join(problems))

    def effective(self) -> "RunConfig":
        """--quick: first two widths, the largest requested cluster, 2/5/1 warm-up/iterations/trials."""
        if not self.quick:
            return self
        return replace(self, n_values=self.n_values[:2], cluster_sizes=(max(self.cluster_sizes),), warmup=2,
                       iterations=5, trials=1)


def run_checked(command: list[str], *, cwd: Path | None = None, timeout: int | None = None):
    result = subprocess.run(command, cwd=cwd, text=True, capture_output=True, timeout=timeout, check=False)
    if result.returncode != 0:
        raise RuntimeError(f"command failed ({result.returncode}): {' '.join(command)}\n"
                           f"stdout:\n{result.stdout}\nstderr:\n{result.stderr}")
    return result


def write_csv(path: Path, rows: list[dict[str, Any]]) -> None:
    """One CSV file from a list of records. The header is the union of the records' keys in order
    of first appearance (records of one table may carry different optional columns); nothing is
    written for an empty table."""
    if not rows:
        return
    header: dict[str, None] = {}
    for record in rows:
        header.update(dict.fromkeys(record))
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("w", newline="", encoding="utf-8") as out:
        writer = csv.DictWriter(out, fieldnames=list(header), restval="")
        writer.writeheader()
        writer.writerows(rows)


def summarize(samples: Iterable[float]) -> dict[str, float]:
    """Median and the 20th / 80th percentiles of the finite samples, the three statistics the
    reference reports for every timing (`dsmem_eval/runner.py:143-151`)."""
    p20, median, p80 = quantiles(list(samples), (0.2, 0.5, 0.8))
    return {"median": median, "p20": p20, "p80": p80}


def safe_ratio(numerator: float, denominator: float) -> float:
    """numerator / denominator, NaN unless both are finite and the denominator is positive."""
    ok = math.isfinite(numerator) and math.isfinite(denominator) and denominator > 0
    return numerator / denominator if ok else math.nan


def benchmark_callable(function, warmup: int, iterations: int, trials: int) -> list[float]:
    """ms per call over `trials` event-timed batches of `iterations` calls (the role of the
    reference's benchmark_callable, runner.py:166-182)."""
    return event_timed_batches(function, warmup, iterations, trials)


def assert_outputs_close(name: str, outputs, references, atol: float, rtol: float) -> list[dict[str, float | int]]:
    """The reference's acceptance rule (runner.py:185-223): int8 outputs may differ by one at a rate
    of at most 1e-5, everything else must pass allclose(atol, rtol). Returns its diagnostics."""
    import torch

    if len(outputs) != len(references):
        raise RuntimeError(f"{name}: output count {len(outputs)} != reference count {len(references)}")
    diagnostics: list[dict[str, float | int]] = []
    for index, (output, reference) in enumerate(zip(outputs, references)):
        if output.dtype == torch.int8:
            difference = (output.to(torch.int16) - reference.to(torch.int16)).abs()
            mismatch = int(torch.count_nonzero(difference).item())
            maximum = int(difference.max().item()) if difference.numel() else 0
            rate = mismatch / max(output.numel(), 1)
            if maximum > 1 or rate > 1.0e-5:
                raise RuntimeError(f"{name} output {index}: {mismatch} int8 mismatches ({rate:.3e}), "
                                   f"maximum difference {maximum}")
            diagnostics.append({"mismatch_count": mismatch, "mismatch_rate": rate, "max_integer_difference": maximum})
            continue
        reference = reference.to(output.dtype).reshape(output.shape)
        max_error = float((output.float() - reference.float()).abs().max().item()) if output.numel() else 0.0
        diagnostics.append({"max_abs_error": max_error})
        if not torch.allclose(output, reference, atol=atol, rtol=rtol):
            raise RuntimeError(f"{name} output {index}: max error {max_error} exceeds atol={atol}, rtol={rtol}")
    return diagnostics


def benchmark_native(name: str, rows: int, cols: int, warmup: int, iterations: int, trials: int,
                     cluster_size: int = 0, opts: dict | None = None) -> dict[str, Any]:
    """In-process arm (the native counterpart of benchmark_frameworks, runner.py:350-441): seeded
    inputs of the registry on cuda:0, one launcher from NATIVE_LAUNCHERS, event timing."""
    import torch

    from .launchers import NATIVE_LAUNCHERS, allocate_outputs

    spec = WORKLOADS[name]
    inputs = spec.input_factory(rows, cols, torch.device("cuda:0"), seed=1234 + cols)
    outputs = allocate_outputs(name, inputs)
    launcher = NATIVE_LAUNCHERS[name]
    samples = benchmark_callable(lambda: launcher(inputs, outputs, cluster_size, dict(opts or {})), warmup, iterations,
                                 trials)
    stats = summarize(samples)
    return {"workload": name, "framework": "native", "rows": rows, "cols": cols, "cluster_size": cluster_size,
            "ms": stats["median"], "p20_ms": stats["p20"], "p80_ms": stats["p80"],
            "gbps": spec.algorithmic_bytes(rows, cols) / stats["median"] / 1.0e6, "samples": samples}


def require_binaries(bin_dir: Path, selected: tuple[str, ...]) -> None:
    required = ["primitive_benchmark", "cluster_control", *selected]
    missing = [name for name in required if not (bin_dir / name).is_file()]
    if missing:
        raise FileNotFoundError(f"missing executables in {bin_dir}: {', '.join(missing)}; "
                                "run `python -m credit_b200.build` first")


def parse_cuda_output(output: str) -> list[dict[str, Any]]:
    """RESULT,cols,rows,block_variant,block_ms,block_gbps,cluster_variant,cluster_ms,cluster_gbps,P,ratio"""
    parsed = []
    for line in output.splitlines():
        if not line.startswith("RESULT,"):
            continue
        f = next(csv.reader([line]))
        parsed.append({
            "cols": int(f[1]), "rows": int(f[2]),
            "block_variant": f[3], "block_ms": math.nan if f[4] == "n/a" else float(f[4]),
            "cluster_variant": f[6], "cluster_ms": math.nan if f[7] == "n/a" else float(f[7]),
            "cluster_size": int(f[9]),
        })
    if not parsed:
        raise RuntimeError(f"workload produced no RESULT rows:\n{output}")
    return parsed


def parse_meta(output: str) -> dict[str, str]:
    meta = {}
    for line in output.splitlines():
        if line.startswith("META,"):
            _, key, value = line.split(",", 2)
            meta[key] = value
    return meta


def run_cuda_trials(name: str, bin_dir: Path, rows: int, n_values: tuple[int, ...], cluster_size: int,
                    warmup: int, iterations: int, trials: int) -> list[dict[str, Any]]:
    command = [str(bin_dir / name), "--csv", "--n-values", ",".join(map(str, n_values)), "--warmup", str(warmup),
               "--iters", str(iterations), "--cluster-size", str(cluster_size)]
    if rows > 0:
        command += ["--rows", str(rows)]
    all_rows = []
    for trial in range(trials):
        output = run_checked(command, timeout=30 * 60).stdout
        meta = parse_meta(output)
        for row in parse_cuda_output(output):
            row["trial"] = trial
            row["dtype"] = meta.get("dtype", "")
            all_rows.append(row)
    return all_rows


def run_control_trials(bin_dir: Path, rows: int, cluster_size: int, barriers: int, shared_bytes: int,
                       warmup: int, iterations: int, trials: int, exchange: str = "mbarrier") -> list[float]:
    command = [str(bin_dir / "cluster_control"), "--rows", str(rows), "--cluster-size", str(cluster_size),
               "--barriers", str(barriers), "--shared-bytes", str(shared_bytes), "--warmup", str(warmup),
               "--iters", str(iterations), "--exchange", exchange]
    samples = []
    for _ in range(trials):
        output = run_checked(command, timeout=10 * 60).stdout
        line = next((ln for ln in output.splitlines() if ln.startswith("CONTROL,")), None)
        if line is None:   # UNSUPPORTED: no samples for this point
            return []
        samples.append(float(line.split(",")[7]))
    return samples


# arrays of the element type a workload stages / writes per row (int8 output of fp32 input: 0.25)
_ARRAYS = {"rmsnorm_forward": (1, 1.0), "row_reduce": (1, 0.0), "layernorm_forward": (1, 1.0),
           "layernorm_backward": (2, 1.0), "layernorm_backward_stats": (2, 1.0), "weighted_var_backward": (3, 1.0),
           "pearson_backward": (2, 2.0), "softmax_logits_backward": (2, 1.0), "lars_momentum": (3, 2.0),
           "rowwise_quant": (1, 0.25)}
_ROW_OPS = ("weighted_var_backward", "pearson_backward", "softmax_logits_backward", "lars_momentum", "rowwise_quant")
WS_THREADS = (352, 608)   # CTA sizes of the warp-specialised kernels


def resident_clusters(name: str, rows: int, cols: int, dtype: str, cluster_size: int) -> tuple[int, int, bool, int]:
    """(co-resident clusters, threads per CTA, register path?, ring stages) of the kernel the
    executable's cluster variant launches at this cluster size, from the library's own planner
    (which asks the driver); (0, 0, False, 0) if the shape does not fit this cluster size."""
    from . import _native as N
    try:
        plan = N.plan(_WORKLOAD_IDS[name], rows, cols, N.BF16 if dtype == "bf16" else N.F32,
                      {"cluster_size": cluster_size, "variant": N.VARIANT_CLUSTER_SMEM if cluster_size > 1 else N.VARIANT_AUTO})
    except N.CreditError:
        return 0, 0, False, 0
    return plan.num_clusters, plan.threads, plan.vectors_per_thread > 0, plan.stages


def library_cluster_size(name: str, rows: int, cols: int, dtype: str) -> int:
    """The cluster size the library picks by itself (cluster_size = 0); 0 if it cannot plan the shape."""
    from . import _native as N
    try:
        return N.plan(_WORKLOAD_IDS[name], rows, cols, N.BF16 if dtype == "bf16" else N.F32).cluster_size
    except N.CreditError:
        return 0


def build_summary(config: RunConfig, profile: cost_model.DeviceProfile, calibration: cost_model.B200Calibration,
                  raw_cuda: list[dict[str, Any]], control_samples: dict[tuple[str, int, int], list[float]],
                  residency: dict[tuple[str, int, int], tuple], auto_choice: dict[tuple[str, int], int] | None = None):
    auto_choice = auto_choice or {}
    groups: dict[tuple[str, int, str, int], list[float]] = defaultdict(list)
    block_names: dict[tuple[str, int], set[str]] = defaultdict(set)
    shape_rows: dict[tuple[str, int], int] = {}
    dtypes: dict[str, str] = {}
    for row in raw_cuda:
        name, cols, p = str(row["workload"]), int(row["cols"]), int(row["cluster_size"])
        shape_rows[(name, cols)] = int(row["rows"])
        dtypes[name] = str(row.get("dtype", ""))
        if math.isfinite(float(row["block_ms"])):
            groups[(name, cols, "block", p)].append(float(row["block_ms"]))
            block_names[(name, cols)].add(str(row["block_variant"]))
        if math.isfinite(float(row["cluster_ms"])):
            groups[(name, cols, "cluster", p)].append(float(row["cluster_ms"]))

    summary_rows, cluster_rows = [], []
    block_p = max(config.cluster_sizes)
    for name in config.workloads:
        spec = WORKLOADS[name]
        elem = 4 if dtypes.get(name, "f32") == "f32" else 2
        for cols in config.n_values:
            rows = shape_rows.get((name, cols))
            if rows is None:
                continue
            block = summarize(groups[(name, cols, "block", block_p)])
            alg_bytes = float(spec.algorithmic_bytes(rows, cols))
            if elem == 4 and spec.dtype.itemsize == 2 or elem == 2 and spec.dtype.itemsize == 4:
                alg_bytes = alg_bytes * elem / spec.dtype.itemsize   # run in the other precision
            measured, ref_candidates, b200_predictions = [], [], []
            for p in config.cluster_sizes:
                cluster = summarize(groups[(name, cols, "cluster", p)])
                if not math.isfinite(cluster["median"]):
                    continue
                measured.append((cluster["median"], p))
                control = summarize(control_samples.get((name, cols, p), []))
                row: dict[str, Any] = {
                    "workload": name, "category": spec.category, "rows": rows, "cols": cols, "cluster_size": p,
                    "shared_bytes_per_cta": cost_model.shared_bytes_per_cta(spec, cols, p),
                    "cluster_ms": cluster["median"], "cluster_p20_ms": cluster["p20"],
                    "cluster_p80_ms": cluster["p80"], "control_overhead_ms": control["median"],
                    "achieved_gbps": alg_bytes / cluster["median"] / 1.0e6,
                }
                if math.isfinite(control["median"]) and math.isfinite(block["median"]) and spec.staged_bytes_per_element:
                    est = cost_model.estimate(spec, cols, p, control["median"], profile, block["median"], rows)
                    ref_candidates.append((est.predicted_delta_ms, p, est))
                    row.update({"model_version": cost_model.MODEL_VERSION,
                                "saved_reread_ms": est.saved_reread_ms, "local_replay_ms": est.local_replay_ms,
                                "local_store_residual_ms": est.local_store_residual_ms,
                                "dsmem_store_ms": est.dsmem_store_ms, "predicted_delta_ms": est.predicted_delta_ms,
                                "predicted_profitable": est.predicted_profitable})
                resident, threads, register_path, stages = (*residency.get((name, cols, p), (0, 0)), True, 3)[:4]
                pred = None
                if not spec.staged_bytes_per_element:       # streaming reduction: nothing staged
                    pred = cost_model.predict_streaming_ms(rows, p, alg_bytes, calibration)
                elif resident > 0 and threads in WS_THREADS:
                    arrays_in, arrays_out = _ARRAYS[name]
                    pred = cost_model.predict_ws_ms(rows, cols, p, resident, threads, elem, arrays_in, arrays_out,
                                                    stages, backward=name == "layernorm_backward_stats",
                                                    row_op=name in _ROW_OPS, cal=calibration)
                elif resident > 0:
                    pred = cost_model.predict_cluster_ms(rows, cols, p, resident, threads, alg_bytes,
                                                         len(spec.reductions_per_stage), True, calibration,
                                                         register_path)
                if pred is not None:
                    b200_predictions.append(pred)
                    row.update({"resident_clusters": resident, "register_path": register_path,
                                "b200_predicted_ms": pred.predicted_ms, "b200_row_period_us": pred.row_period_us})
                row["measured_delta_vs_block_ms"] = block["median"] - cluster["median"]
                cluster_rows.append(row)
            if not measured:
                continue
            best_ms, best_p = min(measured)
            ref_delta, ref_p, ref_est = max(ref_candidates, default=(math.nan, 0, None), key=lambda t: t[0])
            b200_p = cost_model.best_cluster_size(b200_predictions) if b200_predictions else 0
            at_predicted = next((ms for ms, p in measured if p == b200_p), math.nan)
            lib_p = int(auto_choice.get((name, cols), 0))
            at_library = next((ms for ms, p in measured if p == lib_p), math.nan)
            profitable = best_ms < block["median"] if math.isfinite(block["median"]) else True
            summary_rows.append({
                "workload": name, "label": spec.label, "category": spec.category, "rows": rows, "cols": cols,
                "block_variant": "+".join(sorted(block_names[(name, cols)])),
                "cuda_nodsmem_ms": block["median"], "cuda_nodsmem_p20_ms": block["p20"],
                "cuda_nodsmem_p80_ms": block["p80"],
                "dsmem_ms": best_ms, "measured_cluster_size": best_p,
                "dsmem_vs_cuda_nodsmem": safe_ratio(block["median"], best_ms),
                "achieved_gbps": alg_bytes / best_ms / 1.0e6,
                "roofline_fraction_measured": alg_bytes / best_ms / 1.0e6 / calibration.hbm_gbps,
                "roofline_fraction_nominal_8tbs": alg_bytes / best_ms / 1.0e6 / 8000.0,
                "predicted_cluster_size": ref_p, "model_version": cost_model.MODEL_VERSION,
                "predicted_delta_ms": ref_delta,
                "predicted_profitable": bool(ref_est and ref_est.predicted_profitable),
                "measured_profitable_vs_cuda": profitable,
                "model_correct": bool(ref_est) and ref_est.predicted_profitable == profitable,
                "b200_model_version": cost_model.B200_MODEL_VERSION,
                "b200_predicted_cluster_size": b200_p,
                "b200_model_picks_measured_best": b200_p == best_p,
                # the predicted size costs at most 5 % more than the best one (run-to-run noise of
                # neighbouring sizes is a few per cent)
                "b200_model_within_5pct": bool(math.isfinite(at_predicted) and at_predicted <= 1.05 * best_ms),
                "measured_ms_at_b200_predicted": at_predicted,
                # what cluster_size = 0 launches (the planner inside the library), scored among the swept sizes
                "library_cluster_size": lib_p,
                "library_picks_measured_best": lib_p == best_p,
                "library_within_5pct": bool(math.isfinite(at_library) and at_library <= 1.05 * best_ms),
                "measured_ms_at_library_choice": at_library,
            })
    return summary_rows, cluster_rows


def run_suite(raw_config: dict[str, Any], output_dir: Path, requested_gpu: str = "local") -> dict[str, Any]:
    """Runs the configured sweep and writes the bundle (metadata.json, primitive_stdout.txt,
    primitive_profile.json, cuda_raw.csv, control_raw.csv, summary.csv, cluster_sweep.csv)."""
    import torch

    config = RunConfig.from_dict(raw_config).effective()
    output_dir.mkdir(parents=True, exist_ok=True)
    require_binaries(BIN_DIR, () if config.profile_only else config.workloads)
    props = torch.cuda.get_device_properties(0)
    metadata: dict[str, Any] = {"status": "running", "requested_gpu": requested_gpu, "device": props.name,
                                "config": asdict(config), "started": time.time(),
                                "models": [cost_model.MODEL_VERSION, cost_model.B200_MODEL_VERSION]}
    (output_dir / "metadata.json").write_text(json.dumps(metadata, indent=2))

    primitive = run_checked([str(BIN_DIR / "primitive_benchmark")], timeout=20 * 60).stdout
    (output_dir / "primitive_stdout.txt").write_text(primitive)
    parsed = parse_primitive_output(primitive)
    profile = make_device_profile(parsed, props)
    calibration = make_b200_calibration(parsed)
    (output_dir / "primitive_profile.json").write_text(json.dumps(
        {"parsed": parsed, "profile": profile_as_dict(profile), "b200_calibration": asdict(calibration)}, indent=2))
    if config.profile_only:
        metadata["status"] = "complete"
        (output_dir / "metadata.json").write_text(json.dumps(metadata, indent=2))
        return metadata

    raw_cuda: list[dict[str, Any]] = []
    control_rows: list[dict[str, Any]] = []
    control_samples: dict[tuple[str, int, int], list[float]] = {}
    residency: dict[tuple[str, int, int], tuple] = {}
    auto_choice: dict[tuple[str, int], int] = {}
    for name in config.workloads:
        spec = WORKLOADS[name]
        for p in config.cluster_sizes:
            print(f"[credit_b200] {name} cluster size {p}", flush=True)
            rows_out = run_cuda_trials(name, BIN_DIR, config.rows, config.n_values, p, config.warmup,
                                       config.iterations, config.trials)
            for row in rows_out:
                row["workload"] = name
            raw_cuda.extend(rows_out)
            write_csv(output_dir / "cuda_raw.csv", raw_cuda)
            for cols in config.n_values:
                rows = next(r["rows"] for r in rows_out if r["cols"] == cols)
                dtype = rows_out[0]["dtype"] or "f32"
                samples = run_control_trials(BIN_DIR, rows, p, spec.barrier_count,
                                             cost_model.shared_bytes_per_cta(spec, cols, p), config.warmup,
                                             config.iterations, config.trials)
                control_samples[(name, cols, p)] = samples
                control_rows.extend({"workload": name, "cols": cols, "cluster_size": p, "delta_ms": s}
                                    for s in samples)
                residency[(name, cols, p)] = resident_clusters(name, rows, cols, dtype, p)
                auto_choice[(name, cols)] = library_cluster_size(name, rows, cols, dtype)
    write_csv(output_dir / "control_raw.csv", control_rows)
    write_csv(output_dir / "plans.csv", [
        {"workload": k[0], "cols": k[1], "cluster_size": k[2], "resident_clusters": v[0], "threads": v[1],
         "register_path": int(v[2]), "stages": v[3], "library_cluster_size": auto_choice.get((k[0], k[1]), 0)}
        for k, v in residency.items()])
    summary_rows, cluster_rows = build_summary(config, profile, calibration, raw_cuda, control_samples, residency,
                                               auto_choice)
    write_csv(output_dir / "summary.csv", summary_rows)
    write_csv(output_dir / "cluster_sweep.csv", cluster_rows)
    (output_dir / "metadata.json").write_text(json.dumps(metadata, indent=2))
    write_report(output_dir)
    hits = sum(1 for r in summary_rows if r["b200_model_picks_measured_best"])
    near = sum(1 for r in summary_rows if r["b200_model_within_5pct"])
    metadata.update({"status": "complete", "finished": time.time(), "points": len(summary_rows),
                     "b200_model_hits": hits, "b200_model_within_5pct": near,
                     "library_hits": sum(1 for r in summary_rows if r["library_picks_measured_best"]),
                     "library_within_5pct": sum(1 for r in summary_rows if r["library_within_5pct"])})
    (output_dir / "metadata.json").write_text(json.dumps(metadata, indent=2))
    return metadata


def rescore_bundle(bundle_dir: Path) -> dict[str, Any]:
    """Re-evaluates both cost models on a saved bundle (no GPU): reads cuda_raw.csv, control_raw.csv,
    plans.csv and primitive_stdout.txt, rewrites summary.csv and cluster_sweep.csv. The counterpart
    of the reference's scripts/rescore_cost_model.py:99-218."""
    from types import SimpleNamespace

    meta = json.loads((bundle_dir / "metadata.json").read_text())
    config = RunConfig(**{k: tuple(v) if isinstance(v, list) else v for k, v in meta["config"].items()})
    parsed = parse_primitive_output((bundle_dir / "primitive_stdout.txt").read_text())
    saved = json.loads((bundle_dir / "primitive_profile.json").read_text())["profile"]
    props = SimpleNamespace(multi_processor_count=saved["sm_count"], L2_cache_size=saved["l2_capacity_bytes"],
                            shared_memory_per_block_optin=saved["max_shared_bytes_per_cta"])
    profile = make_device_profile(parsed, props)
    calibration = make_b200_calibration(parsed)

    def number(text: str) -> float:
        return float(text) if text not in ("", "nan") else math.nan

    with (bundle_dir / "cuda_raw.csv").open(newline="") as f:
        raw_cuda = [{**r, "cols": int(r["cols"]), "rows": int(r["rows"]), "cluster_size": int(r["cluster_size"]),
                     "block_ms": number(r["block_ms"]), "cluster_ms": number(r["cluster_ms"])}
                    for r in csv.DictReader(f)]
    control: dict[tuple[str, int, int], list[float]] = defaultdict(list)
    with (bundle_dir / "control_raw.csv").open(newline="") as f:
        for r in csv.DictReader(f):
            control[(r["workload"], int(r["cols"]), int(r["cluster_size"]))].append(float(r["delta_ms"]))
    residency, auto_choice = {}, {}
    with (bundle_dir / "plans.csv").open(newline="") as f:
        for r in csv.DictReader(f):
            residency[(r["workload"], int(r["cols"]), int(r["cluster_size"]))] = (
                int(r["resident_clusters"]), int(r["threads"]), bool(int(r["register_path"])), int(r.get("stages") or 3))
            auto_choice[(r["workload"], int(r["cols"]))] = int(r.get("library_cluster_size") or 0)
    summary_rows, cluster_rows = build_summary(config, profile, calibration, raw_cuda, control, residency, auto_choice)
    write_csv(bundle_dir / "summary.csv", summary_rows)
    write_csv(bundle_dir / "cluster_sweep.csv", cluster_rows)
    write_report(bundle_dir)
    return {"points": len(summary_rows),
            "b200_model_hits": sum(1 for r in summary_rows if r["b200_model_picks_measured_best"]),
            "b200_model_within_5pct": sum(1 for r in summary_rows if r["b200_model_within_5pct"])}


def main(argv: list[str] | None = None) -> int:
    """Command line with the flag surface of the reference's scripts/run_local.py:49-79."""
    import argparse

    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--workloads", default="all")
    ap.add_argument("--n-values", default=",".join(map(str, DEFAULT_N_VALUES)))
    ap.add_argument("--cluster-sizes", default=",".join(map(str, DEFAULT_CLUSTER_SIZES)))
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iterations", type=int, default=100)
    ap.add_argument("--trials", type=int, default=5)
    ap.add_argument("--rows", type=int, default=0)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--profile-only", action="store_true")
    ap.add_argument("--output-dir", default="results/local")
    ap.add_argument("--rescore", metavar="BUNDLE", help="re-evaluate the cost models on a saved bundle and exit")
    args = ap.parse_args(argv)
    if args.rescore:
        print(json.dumps(rescore_bundle(Path(args.rescore))))
        return 0
    raw = {
        "workloads": CLI_WORKLOADS if args.workloads == "all" else tuple(args.workloads.split(",")),
        "n_values": tuple(int(v) for v in args.n_values.split(",")),
        "cluster_sizes": tuple(int(v) for v in args.cluster_sizes.split(",")),
        "warmup": args.warmup, "iterations": args.iterations, "trials": args.trials, "rows": args.rows,
        "quick": args.quick, "profile_only": args.profile_only,
    }
    meta = run_suite(raw, Path(args.output_dir))
    print(json.dumps({k: meta[k] for k in ("status", "device") if k in meta}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
