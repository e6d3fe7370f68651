"""Merges result bundles of several runs (other GPUs, other kernel versions) into one comparison.

    python -m credit_b200.analyze BUNDLE [BUNDLE ...] [--labels a,b] [--output-dir results/comparison]

Each bundle is a directory `run_suite` wrote (metadata.json, summary.csv, cluster_sweep.csv).
Output, in the role of the reference's scripts/analyze_results.py:142-201
(cross_gpu_points / aggregate / model tables and a report):

  comparison_points.csv     every summary row of every bundle, labelled
  comparison_by_width.csv   per label and row width: points, wins of the cluster variant over the
                            no-cluster one, geometric-mean speed-up, mean roofline fraction
  comparison_models.csv     per label: how often each cluster-size chooser (the reference's
                            profitability model, the B200 row-period model, the library's own
                            planner) agreed with the measurement
  COMPARISON.md             the three tables as text, plus per workload the measured-best cluster
                            size of every label at the widest common width

Bundles of the reference pipeline itself can be merged too: columns this project adds (roofline,
B200 model, library choice) are left empty for them.
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import pandas as pd

_TRUE = {"true", "1", "yes"}


def _flag(series: pd.Series) -> pd.Series:
    return series.astype(str).str.strip().str.lower().isin(_TRUE)


def load_bundle(path: Path, label: str | None = None) -> pd.DataFrame:
    """summary.csv of one bundle with a `label` column (given, or the bundle's device name)."""
    meta_path, summary_path = path / "metadata.json", path / "summary.csv"
    if not summary_path.is_file():
        raise FileNotFoundError(f"{path} is not a result bundle: summary.csv is missing")
    meta = json.loads(meta_path.read_text()) if meta_path.is_file() else {}
    frame = pd.read_csv(summary_path)
    frame.insert(0, "label", label or str(meta.get("device") or path.name))
    frame.insert(1, "bundle", str(path))
    return frame


def geometric_mean(values) -> float:
    logs = [math.log(v) for v in values if isinstance(v, (int, float)) and v > 0 and math.isfinite(v)]
    return math.exp(sum(logs) / len(logs)) if logs else math.nan


def by_width(points: pd.DataFrame) -> pd.DataFrame:
    rows = []
    for (label, cols), group in points.groupby(["label", "cols"], sort=True):
        speedup = group["dsmem_vs_cuda_nodsmem"] if "dsmem_vs_cuda_nodsmem" in group else pd.Series(dtype=float)
        roof = group["roofline_fraction_measured"] if "roofline_fraction_measured" in group else pd.Series(dtype=float)
        rows.append({"label": label, "cols": int(cols), "points": len(group),
                     "cluster_wins": int((speedup > 1.0).sum()),
                     "geomean_cluster_speedup": geometric_mean(speedup.tolist()),
                     "mean_roofline_fraction": float(roof.mean()) if len(roof.dropna()) else math.nan})
    return pd.DataFrame(rows)


def model_scores(points: pd.DataFrame) -> pd.DataFrame:
    choosers = {"reference_model_sign_correct": "model_correct",
                "b200_model_picks_best": "b200_model_picks_measured_best",
                "b200_model_within_5pct": "b200_model_within_5pct",
                "library_picks_best": "library_picks_measured_best",
                "library_within_5pct": "library_within_5pct"}
    rows = []
    for label, group in points.groupby("label", sort=True):
        row = {"label": label, "points": len(group)}
        for name, column in choosers.items():
            row[name] = int(_flag(group[column]).sum()) if column in group and group[column].notna().any() else None
        rows.append(row)
    return pd.DataFrame(rows)


def best_sizes(points: pd.DataFrame) -> tuple[int, pd.DataFrame]:
    """Measured-best cluster size per workload and label at the widest width every label has."""
    widths = [set(g["cols"].astype(int)) for _, g in points.groupby("label")]
    common = set.intersection(*widths) if widths else set()
    if not common:
        raise ValueError("the bundles have no row width in common")
    width = max(common)
    at = points[points["cols"].astype(int) == width]
    table = at.pivot_table(index="workload", columns="label", values="measured_cluster_size", aggfunc="first")
    return width, table


def _markdown(frame: pd.DataFrame) -> str:
    if frame.empty:
        return "(no rows)\n"
    def cell(v):
        if isinstance(v, float):
            return "" if math.isnan(v) else f"{v:.3f}"
        return "" if v is None else str(v)
    header = "| " + " | ".join(map(str, frame.columns)) + " |"
    rule = "|" + "---|" * len(frame.columns)
    body = ["| " + " | ".join(cell(v) for v in row) + " |" for row in frame.itertuples(index=False)]
    return "\n".join([header, rule, *body]) + "\n"


def analyze(bundles: list[Path], labels: list[str] | None, output_dir: Path) -> dict:
    if labels is not None and len(labels) != len(bundles):
        raise ValueError("one label per bundle")
    frames = [load_bundle(p, labels[i] if labels else None) for i, p in enumerate(bundles)]
    seen = [f["label"].iloc[0] for f in frames if len(f)]
    if len(set(seen)) != len(seen):
        raise ValueError(f"labels must be unique, got {seen} (use --labels)")
    points = pd.concat(frames, ignore_index=True, sort=False)
    widths, models = by_width(points), model_scores(points)
    width, sizes = best_sizes(points)
    output_dir.mkdir(parents=True, exist_ok=True)
    points.to_csv(output_dir / "comparison_points.csv", index=False)
    widths.to_csv(output_dir / "comparison_by_width.csv", index=False)
    models.to_csv(output_dir / "comparison_models.csv", index=False)
    text = ["# Comparison of result bundles\n", "## Per row width\n", _markdown(widths),
            "\n## Cluster-size choosers against the measurement\n", _markdown(models),
            f"\n## Measured-best cluster size at {width} columns\n", _markdown(sizes.reset_index())]
    (output_dir / "COMPARISON.md").write_text("\n".join(text), encoding="utf-8")
    return {"labels": seen, "points": len(points), "common_width": width}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("bundles", nargs="+", type=Path)
    ap.add_argument("--labels", default=None, help="comma-separated, one per bundle (default: the device names)")
    ap.add_argument("--output-dir", type=Path, default=Path("results/comparison"))
    args = ap.parse_args(argv)
    result = analyze([p.resolve() for p in args.bundles], args.labels.split(",") if args.labels else None,
                     args.output_dir)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
