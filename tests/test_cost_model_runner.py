"""CPU tests of the caller side: profile parser, both cost models, the pipeline's
parsers and its summary, on recorded tool output (no GPU, no subprocess).

The arithmetic checks of `estimate` follow the reference's own
tests/test_cost_model.py (hand-computed terms of the same formula)."""
import math
from pathlib import Path
from types import SimpleNamespace

import pytest

from credit_b200 import cost_model, runner
from credit_b200.profile import make_b200_calibration, make_device_profile, parse_primitive_output
from credit_b200.workloads import WORKLOADS

GOLDEN = Path(__file__).parent / "golden"
PROPS = SimpleNamespace(multi_processor_count=148, L2_cache_size=126 * 1024 * 1024,
                        shared_memory_per_block_optin=232448)


@pytest.fixture(scope="module")
def parsed():
    return parse_primitive_output((GOLDEN / "primitive_benchmark_b200.txt").read_text())


def test_parse_primitive_output(parsed):
    assert parsed["name"] == "NVIDIA B200"
    assert parsed["sm_count"] == 148
    assert parsed["clock_ghz"] == pytest.approx(1.97)
    assert parsed["dram_bandwidth_gbps"] == pytest.approx(5954.43)
    assert parsed["cluster_sync_cycles"] == pytest.approx(433.75)
    assert parsed["dsmem_store_bytes_per_cycle_cta"] == pytest.approx(20.53)
    assert sorted(parsed["per_cluster"]) == [2, 4, 8, 16]
    assert parsed["per_cluster"][8]["mbarrier_exchange_cycles"] == pytest.approx(350.64)
    assert parsed["per_cluster"][16]["barrier_exchange_cycles"] == pytest.approx(1059.40)
    assert parsed["bulk_copy_latency_cycles"]
    # cp.async.bulk between the shared memories of two CTAs: cycles per step, bytes per cycle and CTA
    assert parsed["dsmem_bulk_copy"][8][16384] == pytest.approx((1149.17, 17.78))
    assert sorted(parsed["dsmem_bulk_copy"]) == [2, 8, 16]


def test_parse_primitive_output_missing_line(parsed):
    text = (GOLDEN / "primitive_benchmark_b200.txt").read_text().replace("Cluster sync latency ", "Cluster xx latency ")
    with pytest.raises(RuntimeError, match="cluster synchronization latency"):
        parse_primitive_output(text)


def test_device_profile(parsed):
    profile = make_device_profile(parsed, PROPS)
    assert profile.sm_count == 148
    assert profile.l2_bandwidth_gbps == pytest.approx(8776.75 * 1.97)
    assert profile.local_smem_store_bytes_per_cycle_cta == pytest.approx(64.03)
    assert profile.max_shared_bytes_per_cta == 232448


def test_reference_model_terms(parsed):
    profile = make_device_profile(parsed, PROPS)
    spec = WORKLOADS["layernorm_backward"]
    rows, cols, p = 2048, 65536, 8
    est = cost_model.estimate(spec, cols, p, control_overhead_ms=0.01, profile=profile, baseline_ms=0.6, rows=rows)
    assert est.saved_reread_ms == pytest.approx(0.6 * spec.reread_bytes_per_element / spec.modeled_bytes_per_element)
    waves = math.ceil(rows / (148 // p))
    slice_bytes = cols // p * spec.staged_bytes_per_element
    cycles_to_ms = 1.0 / (1.97 * 1.0e6)
    assert est.local_replay_ms == pytest.approx(waves * slice_bytes / 288.07 * cycles_to_ms)
    assert est.dsmem_store_ms == pytest.approx(waves * 4.0 * (p - 1) * spec.partial_count / 20.53 * cycles_to_ms)
    assert est.predicted_delta_ms == pytest.approx(
        est.saved_reread_ms - 0.01 - est.local_replay_ms - est.local_store_residual_ms - est.dsmem_store_ms)
    assert est.predicted_profitable == (est.predicted_delta_ms > 0)
    assert est.local_staging_ms == pytest.approx(est.local_replay_ms + est.local_store_residual_ms)


def test_reference_model_rejects_bad_baseline(parsed):
    profile = make_device_profile(parsed, PROPS)
    with pytest.raises(ValueError):
        cost_model.estimate(WORKLOADS["layernorm_backward"], 4096, 2, 0.0, profile, float("nan"))
    with pytest.raises(ValueError):
        cost_model.estimate(WORKLOADS["row_reduce"], 4096, 2, 0.0, profile, 0.0)


def test_b200_model(parsed):
    cal = make_b200_calibration(parsed)
    assert cal.exchange(8) == pytest.approx(350.64)
    assert cal.exchange(1) < cal.exchange(2)
    rows, cols = 2048, 262144
    alg = rows * cols * 6.0
    small = cost_model.predict_cluster_ms(rows, cols, 2, 70, 512, alg, 1, True, cal)
    wide = cost_model.predict_cluster_ms(rows, cols, 8, 15, 512, alg, 1, True, cal)
    assert small.predicted_ms >= small.hbm_ms and wide.predicted_ms >= wide.hbm_ms
    assert wide.rows_per_cluster == math.ceil(rows / 15)
    assert cost_model.best_cluster_size([small, wide]) in (2, 8)
    # few rows, few resident clusters: the latency chain dominates and the prediction grows with rows
    a = cost_model.predict_cluster_ms(4096, 4096, 8, 15, 256, 4096 * 4096 * 6.0, 2, True, cal)
    b = cost_model.predict_cluster_ms(8192, 4096, 8, 15, 256, 8192 * 4096 * 6.0, 2, True, cal)
    assert b.predicted_ms > a.predicted_ms > a.hbm_ms
    one_shot = cost_model.predict_cluster_ms(4096, 4096, 8, 15, 256, 4096 * 4096 * 6.0, 2, False, cal)
    assert one_shot.predicted_ms > a.predicted_ms
    with pytest.raises(ValueError):
        cost_model.predict_cluster_ms(0, 4096, 8, 15, 256, 1.0, 1)
    with pytest.raises(ValueError):
        cost_model.best_cluster_size([])


def test_warp_specialised_row_period_model():
    """predict_ws_ms on hand-computed cases (the planner's predicted_ws_ms in launch.cu is the same
    formula with the same constants)."""
    cal = cost_model.B200Calibration()
    # C4: bf16 8192 x 65536, P = 8, 15 resident clusters, 6 stages: the output warps' issue time for
    # 32 elements per thread is just above the CTA's share of HBM
    p = cost_model.predict_ws_ms(8192, 65536, 8, 15, 352, 2, 2, 1, 6, backward=True, cal=cal)
    per_sm = cal.hbm_gbps / 120
    hbm_us = 3 * 8192 * 2 / (per_sm * 1e3)
    issue_us = (cal.ws_fixed_cycles + cal.ws_cycles_per_element_bwd * 32) / (cal.clock_ghz * 1e3)
    assert issue_us > hbm_us > 0.9 * issue_us
    assert p.row_period_us == pytest.approx(issue_us) and p.rows_per_cluster == math.ceil(8192 / 15)
    assert p.predicted_ms == pytest.approx(issue_us * (p.rows_per_cluster + cal.ws_fill_rows) * 1e-3)
    assert 0.48 < p.predicted_ms < 0.56        # measured 0.487 burst, 0.553 sustained
    # a short slice in a shallow ring: the loads in flight bound the row period (3 of 6 stages)
    q = cost_model.predict_ws_ms(2048, 16384, 8, 15, 352, 4, 2, 1, 6, cal=cal)
    assert q.row_period_us == pytest.approx(cal.ws_load_latency_us / 3)
    # three stages: two between the passes, one in flight, and the short-ring factor on top
    r = cost_model.predict_ws_ms(2048, 65536, 8, 15, 352, 4, 2, 1, 3, cal=cal)
    assert r.row_period_us == pytest.approx(max(3 * 8192 * 4 / (per_sm * 1e3), cal.ws_load_latency_us) * cal.ws_short_ring_penalty)
    # clusters of 16 carry their measured penalty
    s16 = cost_model.predict_ws_ms(4096, 131072, 16, 7, 352, 2, 1, 1, 8, cal=cal)
    s8 = cost_model.predict_ws_ms(4096, 131072, 8, 15, 352, 2, 1, 1, 6, cal=cal)
    assert s16.predicted_ms > s8.predicted_ms
    with pytest.raises(ValueError):
        cost_model.predict_ws_ms(0, 4096, 8, 15, 352, 2, 1, 1, 6)


def test_planner_rule_restated_in_python():
    """cost_model.ws_plan_rule at shapes whose library plans are known from B200 runs (the GPU suite
    compares the two over the whole sweep)."""
    rule = cost_model.ws_plan_rule
    assert rule("layernorm_backward_stats", 65536, 2, 2, column_sums=True) == (8, 6)     # C4
    assert rule("layernorm_forward", 131072, 2, 1) == (8, 6)                             # C3
    assert rule("layernorm_backward", 65536, 4, 2) == (8, 3)        # 16 never replaces an 8 that fits
    assert rule("layernorm_backward", 8192, 4, 2) == (2, 6)         # P = 1 would have three stages only
    assert rule("layernorm_forward", 4096, 2, 1) == (1, 8)          # short slice: 8 stages in half the shared memory
    assert rule("lars_momentum", 16384, 4, 3) == (8, 6)             # LARS wants six stages
    assert rule("weighted_var_backward", 65536, 4, 3) == (16, 4)
    assert rule("pearson_backward", 16384, 4, 2) == (4, 6)
    assert rule("layernorm_forward", 1 << 21, 2, 1) is None         # no slice fits the output threads
    with pytest.raises(ValueError):
        rule("layernorm_forward", 0, 2, 1)


def test_best_cluster_size_prefers_smaller_on_tie():
    p = [cost_model.ClusterPrediction(8, 1.0, 1, 1.0, 1.0), cost_model.ClusterPrediction(4, 1.0, 1, 1.0, 1.0)]
    assert cost_model.best_cluster_size(p) == 4


CLI_OUTPUT = """META,device_name,NVIDIA B200
META,workload,layernorm_backward
META,dtype,f32
RESULT,4096,2048,block_smem,0.0300,3355.4,cluster_smem,0.0250,4026.5,8,1.200
RESULT,65536,2048,block_read,0.6000,3579.1,cluster_smem,0.3750,5726.6,8,1.600
RESULT,131072,2048,n/a,n/a,n/a,cluster_smem,0.8000,5368.7,8,n/a
"""


def test_parse_cuda_output():
    rows = runner.parse_cuda_output(CLI_OUTPUT)
    assert [r["cols"] for r in rows] == [4096, 65536, 131072]
    assert rows[1]["block_variant"] == "block_read" and rows[1]["block_ms"] == pytest.approx(0.6)
    assert math.isnan(rows[2]["block_ms"]) and rows[2]["cluster_ms"] == pytest.approx(0.8)
    assert all(r["cluster_size"] == 8 and r["rows"] == 2048 for r in rows)
    assert runner.parse_meta(CLI_OUTPUT)["dtype"] == "f32"
    with pytest.raises(RuntimeError):
        runner.parse_cuda_output("META,device_name,x\n")


def test_run_config_validation():
    cfg = runner.RunConfig.from_dict({"workloads": ["row_reduce"], "cluster_sizes": [2, 16], "quick": True})
    eff = cfg.effective()
    assert eff.cluster_sizes == (16,) and eff.n_values == runner.DEFAULT_N_VALUES[:2]
    assert (eff.warmup, eff.iterations, eff.trials) == (2, 5, 1)
    for bad in ({"workloads": ["softmax"]}, {"cluster_sizes": [3]}, {"n_values": [0]}, {"trials": 0}, {"rows": -1}):
        with pytest.raises(ValueError):
            runner.RunConfig.from_dict(bad)


def test_summarize_and_percentile():
    s = runner.summarize([1.0, 2.0, 3.0, 4.0, float("nan")])
    assert s["median"] == pytest.approx(2.5)
    assert s["p20"] == pytest.approx(1.6) and s["p80"] == pytest.approx(3.4)
    assert math.isnan(runner.summarize([])["median"])
    assert math.isnan(runner.safe_ratio(1.0, 0.0))


def test_build_summary(parsed):
    profile = make_device_profile(parsed, PROPS)
    cal = make_b200_calibration(parsed)
    cfg = runner.RunConfig(workloads=("layernorm_backward",), n_values=(65536,), cluster_sizes=(4, 8), trials=2)
    raw, control, residency = [], {}, {}
    for p, ms in ((4, 0.45), (8, 0.375)):
        for trial in range(2):
            raw.append({"workload": "layernorm_backward", "cols": 65536, "rows": 2048, "trial": trial, "dtype": "f32",
                        "block_variant": "block_read", "block_ms": 0.6, "cluster_variant": "cluster_smem",
                        "cluster_ms": ms + 0.001 * trial, "cluster_size": p})
        control[("layernorm_backward", 65536, p)] = [0.01, 0.012]
        residency[("layernorm_backward", 65536, p)] = (148 // p - 3, 512)
    summary, sweep = runner.build_summary(cfg, profile, cal, raw, control, residency)
    assert len(summary) == 1 and len(sweep) == 2
    row = summary[0]
    assert row["measured_cluster_size"] == 8
    assert row["dsmem_ms"] == pytest.approx(0.3755)
    assert row["dsmem_vs_cuda_nodsmem"] == pytest.approx(0.6 / 0.3755)
    assert row["measured_profitable_vs_cuda"] is True
    assert row["predicted_cluster_size"] in (4, 8) and row["b200_predicted_cluster_size"] in (4, 8)
    assert 0.0 < row["roofline_fraction_measured"] < 1.2
    assert {"saved_reread_ms", "b200_predicted_ms", "control_overhead_ms"} <= set(sweep[0])


def test_require_binaries_names_what_is_missing(tmp_path):
    with pytest.raises(FileNotFoundError, match="cluster_control"):
        runner.require_binaries(tmp_path, ("row_reduce",))


def test_generic_path_and_streaming_predictions(parsed):
    cal = make_b200_calibration(parsed)
    alg = 8192 * 65536 * 6.0
    reg = cost_model.predict_cluster_ms(8192, 65536, 8, 15, 512, alg, 1, True, cal, register_path=True)
    gen = cost_model.predict_cluster_ms(8192, 65536, 2, 74, 256, alg, 1, True, cal, register_path=False)
    assert gen.predicted_ms == pytest.approx(gen.hbm_ms / cal.generic_path_efficiency)
    assert cost_model.best_cluster_size([gen, reg]) == 8      # the re-read kernels lose to the register path
    # streaming reduction: few CTAs cannot fill HBM, many CTAs cost launch time
    few = cost_model.predict_streaming_ms(16, 2, 16 * 1048576 * 4.0, cal)
    many = cost_model.predict_streaming_ms(16, 16, 16 * 1048576 * 4.0, cal)
    assert many.predicted_ms < few.predicted_ms
    tiny2 = cost_model.predict_streaming_ms(512, 2, 512 * 4096 * 4.0, cal)
    tiny16 = cost_model.predict_streaming_ms(512, 16, 512 * 4096 * 4.0, cal)
    assert tiny2.predicted_ms < tiny16.predicted_ms
    with pytest.raises(ValueError):
        cost_model.predict_streaming_ms(0, 2, 1.0, cal)


def test_rescore_bundle_round_trip(tmp_path, parsed):
    """A saved bundle is re-scored offline: same files in, summary and sweep rewritten."""
    import csv
    import json
    from dataclasses import asdict

    cfg = runner.RunConfig(workloads=("layernorm_backward_stats",), n_values=(65536,), cluster_sizes=(2, 8), trials=1)
    (tmp_path / "metadata.json").write_text(json.dumps({"config": asdict(cfg)}))
    (tmp_path / "primitive_stdout.txt").write_text((GOLDEN / "primitive_benchmark_b200.txt").read_text())
    profile = make_device_profile(parsed, PROPS)
    (tmp_path / "primitive_profile.json").write_text(json.dumps({"profile": asdict(profile)}))
    raw = [{"workload": "layernorm_backward_stats", "cols": 65536, "rows": 8192, "trial": 0, "dtype": "bf16",
            "block_variant": "block_read", "block_ms": 1.93, "cluster_variant": "cluster_smem", "cluster_ms": ms,
            "cluster_size": p} for p, ms in ((2, 1.84), (8, 0.83))]
    runner.write_csv(tmp_path / "cuda_raw.csv", raw)
    runner.write_csv(tmp_path / "control_raw.csv", [
        {"workload": "layernorm_backward_stats", "cols": 65536, "cluster_size": p, "delta_ms": 0.03} for p in (2, 8)])
    runner.write_csv(tmp_path / "plans.csv", [
        {"workload": "layernorm_backward_stats", "cols": 65536, "cluster_size": 2, "resident_clusters": 74,
         "threads": 256, "register_path": 0, "library_cluster_size": 8},
        {"workload": "layernorm_backward_stats", "cols": 65536, "cluster_size": 8, "resident_clusters": 15,
         "threads": 512, "register_path": 1, "library_cluster_size": 8}])
    result = runner.rescore_bundle(tmp_path)
    assert result == {"points": 1, "b200_model_hits": 1, "b200_model_within_5pct": 1}
    with (tmp_path / "summary.csv").open() as f:
        (row,) = list(csv.DictReader(f))
    assert row["measured_cluster_size"] == "8" and row["b200_predicted_cluster_size"] == "8"
    with (tmp_path / "cluster_sweep.csv").open() as f:
        sweep = list(csv.DictReader(f))
    assert [r["register_path"] for r in sweep] == ["False", "True"]
    report = (tmp_path / "REPORT.md").read_text()
    assert "would pick the measured-best size at 1/1 points" in report and "The library's planner" in report
    assert "| layernorm_backward_stats | 65536 | 1930.0 | 1840.0 | 830.0 | 8 | 8 | 830.0 | yes | 8 |" in report
    assert "planner (what cluster_size = 0 launches: a rule calibrated on B200 sweeps) picks the measured-best cluster size at 1/1" in report
    assert json.loads((tmp_path / "aggregate.json").read_text())["b200_model_within_5pct"] == 1


def test_assert_outputs_close_rules():
    import torch

    a = torch.tensor([1.0, 2.0, 3.0])
    assert runner.assert_outputs_close("w", (a,), (a + 1e-7,), 1e-6, 1e-6)[0]["max_abs_error"] < 1e-6
    with pytest.raises(RuntimeError, match="exceeds"):
        runner.assert_outputs_close("w", (a,), (a + 1e-2,), 1e-6, 1e-6)
    with pytest.raises(RuntimeError, match="output count"):
        runner.assert_outputs_close("w", (a,), (a, a), 1e-6, 1e-6)
    q = torch.zeros(200000, dtype=torch.int8)
    r = q.clone()
    r[0] = 1                                      # one off-by-one in 200k: rate 5e-6 is accepted
    assert runner.assert_outputs_close("q", (q,), (r,), 0, 0)[0]["mismatch_count"] == 1
    r[1] = 2                                      # a difference of two is not
    with pytest.raises(RuntimeError, match="int8 mismatches"):
        runner.assert_outputs_close("q", (q,), (r,), 0, 0)
