"""Markdown report of a result bundle.

Follows the reference's report writer (`dsmem_eval/report.py:29-139`: headline counts,
results at the widest rows, crossover validation) with what this project adds to a
bundle: roofline columns, the predicted against the measured-best cluster size of
the B200 model, and the full per-cluster-size table.
"""
from __future__ import annotations

import csv
import json
import math
from collections import defaultdict
from pathlib import Path
from typing import Any, Iterable


def _truth(value: Any) -> bool:
    return value if isinstance(value, bool) else str(value).strip().lower() == "true"


def _number(value: Any) -> float:
    try:
        return float(value)
    except (TypeError, ValueError):
        return math.nan


def geometric_mean(values: Iterable[float]) -> float:
    positive = [v for v in values if v > 0.0 and math.isfinite(v)]
    return math.exp(sum(math.log(v) for v in positive) / len(positive)) if positive else math.nan


def build_report(summary_rows: list[dict[str, Any]], sweep_rows: list[dict[str, Any]],
                 metadata: dict[str, Any]) -> tuple[str, dict[str, Any]]:
    valid = [r for r in summary_rows if math.isfinite(_number(r.get("dsmem_vs_cuda_nodsmem")))]
    wins = sum(_number(r["dsmem_vs_cuda_nodsmem"]) > 1.0 for r in valid)
    ref_rows = [r for r in summary_rows if "model_correct" in r]
    ref_correct = sum(_truth(r["model_correct"]) for r in ref_rows)
    b200_rows = [r for r in summary_rows if str(r.get("b200_predicted_cluster_size", "0")) not in ("0", "")]
    strict = sum(_truth(r.get("b200_model_picks_measured_best")) for r in b200_rows)
    near = sum(_truth(r.get("b200_model_within_5pct")) for r in b200_rows)
    lib_rows = [r for r in summary_rows if str(r.get("library_cluster_size", "0")) not in ("0", "")]
    lib_strict = sum(_truth(r.get("library_picks_measured_best")) for r in lib_rows)
    lib_near = sum(_truth(r.get("library_within_5pct")) for r in lib_rows)
    widest = max((int(r["cols"]) for r in valid), default=0)
    widest_rows = [r for r in valid if int(r["cols"]) == widest]
    speedup = geometric_mean(_number(r["dsmem_vs_cuda_nodsmem"]) for r in widest_rows)

    by_workload: dict[str, list[dict[str, Any]]] = defaultdict(list)
    for r in summary_rows:
        by_workload[str(r["workload"])].append(r)
    crossovers = []
    for rows in by_workload.values():
        ordered = sorted(rows, key=lambda r: int(r["cols"]))
        measured = next((int(r["cols"]) for r in ordered if _truth(r.get("measured_profitable_vs_cuda"))), None)
        predicted = next((int(r["cols"]) for r in ordered if _truth(r.get("predicted_profitable"))), None)
        crossovers.append({"workload": ordered[0]["workload"], "label": ordered[0].get("label", ordered[0]["workload"]),
                           "predicted": predicted, "measured": measured})

    device = str(metadata.get("device", "unknown device"))
    lines = [
        f"# {device}: cluster / DSMEM evaluation",
        "",
        f"- The cluster kernels beat the faster no-cluster variant on {wins}/{len(valid)} workload-size points.",
        f"- The library's planner (what cluster_size = 0 launches: a rule calibrated on B200 sweeps) picks the "
        f"measured-best cluster size at {lib_strict}/{len(lib_rows)} points; its pick costs at most 5 % more than the "
        f"best size at {lib_near}/{len(lib_rows)}.",
        f"- The B200 row-period model (a time predictor; the planner no longer chooses by it) would pick the "
        f"measured-best size at {strict}/{len(b200_rows)} points, within 5 % at {near}/{len(b200_rows)}.",
        f"- The reference's profitability model predicts {ref_correct}/{len(ref_rows)} profitability signs correctly.",
    ]
    if widest:
        lines.append(f"- At N={widest} the cluster kernels are {speedup:.3f}x (geometric mean) the no-cluster variants.")
    lines += ["", f"## Results at N={widest}", "",
              "| Workload | rows | block ms | cluster ms | cluster / block | P | GB/s | of measured HBM | planner P | model P |",
              "|---|---:|---:|---:|---:|---:|---:|---:|---:|---:|"]
    for r in widest_rows:
        lines.append(
            f"| {r.get('label', r['workload'])} | {r['rows']} | {_number(r['cuda_nodsmem_ms']):.4f} "
            f"| {_number(r['dsmem_ms']):.4f} | {_number(r['dsmem_vs_cuda_nodsmem']):.3f}x | {r['measured_cluster_size']} "
            f"| {_number(r['achieved_gbps']):.0f} | {_number(r['roofline_fraction_measured']):.2f} "
            f"| {r.get('library_cluster_size', '')} | {r.get('b200_predicted_cluster_size', '')} |")
    lines += ["", "## Crossover validation", "",
              "First width at which clusters beat the faster no-cluster variant (reference model: predicted).", "",
              "| Workload | Predicted | Measured |", "|---|---:|---:|"]
    for c in crossovers:
        lines.append(f"| {c['label']} | {c['predicted'] or 'none'} | {c['measured'] or 'none'} |")

    sweep: dict[tuple[str, str], dict[int, dict[str, Any]]] = defaultdict(dict)
    sizes: set[int] = set()
    for r in sweep_rows:
        sweep[(str(r["workload"]), str(r["cols"]))][int(r["cluster_size"])] = r
        sizes.add(int(r["cluster_size"]))
    ordered_sizes = sorted(sizes)
    lines += ["", "## All points (times in microseconds; n/a: the variant does not fit)", "",
              "| workload | N | block | " + " | ".join(f"P={p}" for p in ordered_sizes) +
              " | best P | planner P | time at planner P | within 5 % | model P |",
              "|---|---:|---:|" + "---:|" * len(ordered_sizes) + "---:|---:|---:|---|---:|"]
    for r in summary_rows:
        cells = []
        for p in ordered_sizes:
            c = sweep.get((str(r["workload"]), str(r["cols"])), {}).get(p)
            cells.append(f"{_number(c['cluster_ms']) * 1000:.1f}" if c else "n/a")
        block = _number(r["cuda_nodsmem_ms"]) * 1000
        at_pred = _number(r.get("measured_ms_at_library_choice")) * 1000
        lines.append(
            f"| {r['workload']} | {r['cols']} | {'n/a' if math.isnan(block) else f'{block:.1f}'} | " + " | ".join(cells) +
            f" | {r['measured_cluster_size']} | {r.get('library_cluster_size', '')} "
            f"| {'n/a' if math.isnan(at_pred) else f'{at_pred:.1f}'} "
            f"| {'yes' if _truth(r.get('library_within_5pct')) else 'no'} | {r.get('b200_predicted_cluster_size', '')} |")

    errors = sorted(abs(_number(r["b200_predicted_ms"]) / _number(r["cluster_ms"]) - 1.0) for r in sweep_rows
                    if _truth(r.get("register_path")) and math.isfinite(_number(r.get("b200_predicted_ms"))))
    if errors:
        lines += ["", f"Predicted against measured time over the {len(errors)} register-path points: median error "
                      f"{100 * errors[len(errors) // 2]:.0f} %, 90th percentile {100 * errors[int(len(errors) * 0.9)]:.0f} %."]
    aggregate = {
        "device": device, "points": len(valid), "wins_over_block": wins,
        "reference_model_points": len(ref_rows), "reference_model_correct": ref_correct,
        "b200_model_points": len(b200_rows), "b200_model_strict": strict, "b200_model_within_5pct": near,
        "library_points": len(lib_rows), "library_strict": lib_strict, "library_within_5pct": lib_near,
        "largest_width": widest, "largest_width_geomean_speedup": speedup, "crossovers": crossovers,
    }
    return "\n".join(lines) + "\n", aggregate


def _read_csv(path: Path) -> list[dict[str, Any]]:
    if not path.exists():
        return []
    with path.open(newline="", encoding="utf-8") as f:
        return list(csv.DictReader(f))


def write_report(bundle_dir: Path) -> dict[str, Any]:
    """Writes REPORT.md and aggregate.json into a bundle from its summary.csv, cluster_sweep.csv
    and metadata.json."""
    bundle_dir = Path(bundle_dir)
    metadata = json.loads((bundle_dir / "metadata.json").read_text()) if (bundle_dir / "metadata.json").exists() else {}
    report, aggregate = build_report(_read_csv(bundle_dir / "summary.csv"), _read_csv(bundle_dir / "cluster_sweep.csv"),
                                     metadata)
    (bundle_dir / "REPORT.md").write_text(report, encoding="utf-8")
    (bundle_dir / "aggregate.json").write_text(json.dumps(aggregate, indent=2), encoding="utf-8")
    return aggregate
