"""Cross-bundle analysis (`python -m credit_b200.analyze`), the role of the reference's
scripts/analyze_results.py: two saved bundles in, comparison tables and a report out."""
import json

import pandas as pd
import pytest

from credit_b200 import analyze


def write_bundle(path, device, rows):
    path.mkdir()
    (path / "metadata.json").write_text(json.dumps({"device": device, "status": "complete"}))
    pd.DataFrame(rows).to_csv(path / "summary.csv", index=False)


def row(workload, cols, best_p, speedup, roof, ref_ok, b200_ok, lib_ok):
    return {"workload": workload, "cols": cols, "rows": 4096, "measured_cluster_size": best_p,
            "dsmem_vs_cuda_nodsmem": speedup, "roofline_fraction_measured": roof, "model_correct": ref_ok,
            "b200_model_picks_measured_best": b200_ok, "b200_model_within_5pct": True,
            "library_picks_measured_best": lib_ok, "library_within_5pct": True}


def test_two_bundles_merge_into_tables_and_a_report(tmp_path):
    a, b = tmp_path / "a", tmp_path / "b"
    write_bundle(a, "NVIDIA B200", [row("pearson_backward", 16384, 4, 1.9, 0.98, True, True, False),
                                    row("pearson_backward", 65536, 8, 2.0, 1.0, True, True, True),
                                    row("lars_momentum", 65536, 16, 1.6, 1.04, False, True, True)])
    write_bundle(b, "NVIDIA H100", [row("pearson_backward", 65536, 8, 1.3, 0.7, True, False, False),
                                    row("lars_momentum", 65536, 8, 0.9, 0.6, True, False, False)])
    out = tmp_path / "cmp"
    result = analyze.analyze([a, b], None, out)
    assert result == {"labels": ["NVIDIA B200", "NVIDIA H100"], "points": 5, "common_width": 65536}
    widths = pd.read_csv(out / "comparison_by_width.csv")
    b200_wide = widths[(widths.label == "NVIDIA B200") & (widths.cols == 65536)].iloc[0]
    assert b200_wide.points == 2 and b200_wide.cluster_wins == 2
    assert b200_wide.geomean_cluster_speedup == pytest.approx((2.0 * 1.6) ** 0.5)
    h100 = widths[widths.label == "NVIDIA H100"].iloc[0]
    assert h100.cluster_wins == 1
    models = pd.read_csv(out / "comparison_models.csv").set_index("label")
    assert models.loc["NVIDIA B200", "reference_model_sign_correct"] == 2
    assert models.loc["NVIDIA B200", "b200_model_picks_best"] == 3 and models.loc["NVIDIA B200", "library_picks_best"] == 2
    assert models.loc["NVIDIA H100", "b200_model_picks_best"] == 0
    report = (out / "COMPARISON.md").read_text()
    assert "Measured-best cluster size at 65536 columns" in report
    assert "| lars_momentum | 16 | 8 |" in report


def test_labels_must_be_unique_and_widths_must_overlap(tmp_path):
    a, b = tmp_path / "a", tmp_path / "b"
    write_bundle(a, "NVIDIA B200", [row("rowwise_quant", 4096, 2, 1.1, 0.5, True, True, True)])
    write_bundle(b, "NVIDIA B200", [row("rowwise_quant", 8192, 2, 1.1, 0.5, True, True, True)])
    with pytest.raises(ValueError, match="unique"):
        analyze.analyze([a, b], None, tmp_path / "o")
    with pytest.raises(ValueError, match="no row width in common"):
        analyze.analyze([a, b], ["first", "second"], tmp_path / "o")
    with pytest.raises(FileNotFoundError):
        analyze.load_bundle(tmp_path / "nothing")
    assert analyze.main([str(a), "--labels", "only", "--output-dir", str(tmp_path / "single")]) == 0
