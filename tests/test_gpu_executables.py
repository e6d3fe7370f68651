"""The process boundary on a GPU: the executables the evaluation pipeline spawns.

The reference pipeline never links a library; it starts `build/<workload>`,
`build/cluster_control` and `build/primitive_benchmark` and reads their stdout
(`dsmem_eval/runner.py:248-347`). These tests start the executables built from this
project with the reference's flags and check what the reference's parsers rely on:
exit codes, the `META,` / `RESULT,` / `CONTROL,` / `UNSUPPORTED,` lines and the
labelled lines of the primitive benchmark. Every workload executable runs with its
in-binary verification ON (a sampled fp64 recomputation on the host, the role of
`verify_selected`, `src/workloads/layernorm_backward.cu:676-705`): a wrong result
is a non-zero exit code.
"""
import csv
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest

from credit_b200 import build, profile, runner

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
BIN = build.BIN_DIR
BLOCK_NAMES = {"block_read", "block_smem"}


@pytest.fixture(scope="module", autouse=True)
def _executables(native_lib):
    build.build_cli()
    runner.require_binaries(BIN, runner.CLI_WORKLOADS)


def spawn(args, timeout=600):
    return subprocess.run([str(a) for a in args], text=True, capture_output=True, timeout=timeout, check=False,
                          cwd=ROOT)


@pytest.mark.parametrize("name", runner.CLI_WORKLOADS)
def test_workload_executable_verifies_and_prints_the_result_protocol(name):
    """`--csv --rows 64 --n-values 4096,4099 --warmup 1 --iters 2 --cluster-size 4`: an aligned and
    a ragged width, verification on. Field order as the reference prints it
    (layernorm_backward.cu:739-758) and reads it (runner.py:263-273: fields 1,2,3,4,6,7,9)."""
    done = spawn([BIN / name, "--csv", "--rows", 64, "--n-values", "4096,4099", "--warmup", 1, "--iters", 2,
                  "--cluster-size", 4])
    assert done.returncode == 0, done.stdout + done.stderr
    meta = runner.parse_meta(done.stdout)
    assert meta["workload"] == name and meta["rows"] == "64"
    assert meta["requested_cluster_size"] == "4" and meta["chosen_cluster_size"] == "4"
    assert meta["dtype"] in ("f32", "bf16") and meta["sm"] == "10.0"

    lines = [ln for ln in done.stdout.splitlines() if ln.startswith("RESULT,")]
    assert len(lines) == 2
    for line, cols in zip(lines, (4096, 4099)):
        f = next(csv.reader([line]))
        assert len(f) == 11, line
        assert (int(f[1]), int(f[2])) == (cols, 64)
        assert f[3] in BLOCK_NAMES and f[6] == "cluster_smem" and int(f[9]) == 4
        block_ms, block_gbps, cluster_ms, cluster_gbps, ratio = (float(f[i]) for i in (4, 5, 7, 8, 10))
        assert min(block_ms, block_gbps, cluster_ms, cluster_gbps) > 0
        assert math.isclose(ratio, block_ms / cluster_ms, rel_tol=1e-3)
    parsed = runner.parse_cuda_output(done.stdout)
    assert [(r["cols"], r["rows"], r["cluster_size"]) for r in parsed] == [(4096, 64, 4), (4099, 64, 4)]
    assert all(math.isfinite(r["block_ms"]) and math.isfinite(r["cluster_ms"]) for r in parsed)


def test_workload_executable_flags_of_the_reference():
    """--batch-size is an alias of --rows, --profile-variant isolates one variant (the other prints
    n/a), --no-verify is accepted, the human-readable table is the default, and a bad flag is
    exit code 1 with `error:` on stderr (layernorm_backward.cu:103-128, 824-827)."""
    exe = BIN / "layernorm_backward"
    only_cluster = spawn([exe, "--csv", "--batch-size", 32, "--n-values", 8192, "--warmup", 1, "--iters", 2,
                          "--cluster-size", 8, "--profile-variant", "cluster", "--no-verify"])
    assert only_cluster.returncode == 0, only_cluster.stderr
    (row,) = runner.parse_cuda_output(only_cluster.stdout)
    assert row["rows"] == 32 and math.isnan(row["block_ms"]) and math.isfinite(row["cluster_ms"])
    only_block = spawn([exe, "--csv", "--rows", 32, "--n-values", 8192, "--warmup", 1, "--iters", 2,
                        "--profile-variant", "block"])
    (row,) = runner.parse_cuda_output(only_block.stdout)
    assert math.isfinite(row["block_ms"]) and math.isnan(row["cluster_ms"])

    human = spawn([exe, "--rows", 32, "--n-values", 4096, "--warmup", 1, "--iters", 2, "--cluster-size", 2])
    assert human.returncode == 0 and "RESULT," not in human.stdout and "cluster" in human.stdout

    bad = spawn([exe, "--no-such-flag"])
    assert bad.returncode == 1 and bad.stderr.startswith("error:")
    bad = spawn([exe, "--profile-variant", "both"])
    assert bad.returncode == 1 and "error:" in bad.stderr
    assert spawn([exe, "--help"]).returncode == 0


def test_row_too_wide_for_a_variant_prints_na_not_an_error():
    """A slice that does not fit shared memory makes the variant n/a, exit code 0
    (layernorm_backward.cu:508-511, 563-565)."""
    done = spawn([BIN / "weighted_var_backward", "--csv", "--rows", 8, "--n-values", 131072, "--warmup", 1,
                  "--iters", 1, "--cluster-size", 2])
    assert done.returncode == 0, done.stderr
    (row,) = runner.parse_cuda_output(done.stdout)
    assert math.isnan(row["cluster_ms"])       # 3 arrays x 256 KiB per CTA cannot be staged
    assert math.isfinite(row["block_ms"])      # the no-staging variant still runs


@pytest.mark.parametrize("exchange", ["barrier", "mbarrier"])
def test_cluster_control_prints_the_control_line(exchange):
    """CONTROL,rows,P,barriers,shared_bytes,block_ms,cluster_ms,delta (cluster_control.cu:171-174);
    the pipeline reads field 7 (runner.py:346)."""
    done = spawn([BIN / "cluster_control", "--rows", 512, "--cluster-size", 8, "--barriers", 2,
                  "--shared-bytes", 32768, "--warmup", 2, "--iters", 5, "--exchange", exchange])
    assert done.returncode == 0, done.stderr
    (line,) = [ln for ln in done.stdout.splitlines() if ln.startswith("CONTROL,")]
    f = line.split(",")
    assert len(f) == 8 and [int(v) for v in f[1:5]] == [512, 8, 2, 32768]
    block_ms, cluster_ms, delta = float(f[5]), float(f[6]), float(f[7])
    assert block_ms > 0 and cluster_ms > 0 and math.isclose(delta, cluster_ms - block_ms, rel_tol=1e-3, abs_tol=1e-6)
    samples = runner.run_control_trials(BIN, 512, 8, 2, 32768, 2, 5, 2, exchange=exchange)
    assert len(samples) == 2 and all(math.isfinite(s) for s in samples)


def test_cluster_control_reports_unsupported_shapes():
    """More shared memory than a CTA can have: one UNSUPPORTED line, exit code 0, and the pipeline
    records no samples for the point (cluster_control.cu:124-130, runner.py:341-345)."""
    done = spawn([BIN / "cluster_control", "--rows", 64, "--cluster-size", 4, "--barriers", 2,
                  "--shared-bytes", 400000, "--warmup", 1, "--iters", 1])
    assert done.returncode == 0
    assert done.stdout.startswith("UNSUPPORTED,64,4,2,400000,") and "CONTROL," not in done.stdout
    assert runner.run_control_trials(BIN, 64, 4, 2, 400000, 1, 1, 1) == []
    bad = spawn([BIN / "cluster_control", "--cluster-size", 3])
    assert bad.returncode == 1 and "error:" in bad.stderr


def test_primitive_benchmark_output_parses_into_a_device_profile():
    """Every labelled line the reference's parser requires (profile.py:33-101), plus the
    per-cluster-size lines of this project's benchmark for P = 2..16."""
    import torch

    done = spawn([BIN / "primitive_benchmark"], timeout=900)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    parsed = profile.parse_primitive_output(done.stdout)
    assert parsed["sm_count"] == torch.cuda.get_device_properties(0).multi_processor_count
    assert 0.5 < parsed["clock_ghz"] < 3.0
    assert parsed["l1_latency_cycles"] < parsed["l2_latency_cycles"] < parsed["dram_latency_cycles"]
    assert parsed["dram_bandwidth_gbps"] > 2000.0
    assert parsed["dsmem_read_latency_cycles"] > parsed["local_smem_read_latency_cycles"] > 0
    assert sorted(parsed["per_cluster"]) == [2, 4, 8, 16]
    for p, entry in parsed["per_cluster"].items():
        assert entry["mbarrier_exchange_cycles"] > 0 and entry["barrier_exchange_cycles"] > 0, p
    # bulk copies between the shared memories of two CTAs of a cluster (cp.async.bulk, completion on the
    # receiver's mbarrier): a step costs more than a DSMEM load, and larger copies move more bytes per cycle
    assert "timed out" not in done.stdout
    for p in (2, 8, 16):
        bulk = parsed["dsmem_bulk_copy"][p]
        assert sorted(bulk) == [256, 1024, 4096, 16384]
        assert bulk[256][0] > parsed["dsmem_read_latency_cycles"] * 0.5
        assert bulk[16384][1] > bulk[256][1] > 0
    device_profile = profile.make_device_profile(parsed, torch.cuda.get_device_properties(0))
    assert device_profile.sm_count == parsed["sm_count"]
    calibration = profile.make_b200_calibration(parsed)
    assert calibration.hbm_gbps > 0


def test_pipeline_quick_run_writes_the_bundle(tmp_path):
    """`python -m credit_b200.runner --quick`: spawns the executables, writes the result bundle of
    the reference pipeline (runner.py:656-793): raw and summary tables, metadata status complete."""
    out = tmp_path / "bundle"
    done = spawn([sys.executable, "-m", "credit_b200.runner", "--quick", "--workloads",
                  "layernorm_backward,rowwise_quant,layernorm_backward_stats", "--n-values", "4096,8192",
                  "--cluster-sizes", "4", "--rows", "256", "--output-dir", out], timeout=1500)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    for name in ("cuda_raw.csv", "control_raw.csv", "summary.csv", "cluster_sweep.csv", "primitive_stdout.txt",
                 "primitive_profile.json", "metadata.json", "REPORT.md"):
        assert (out / name).is_file(), name
    meta = json.loads((out / "metadata.json").read_text())
    assert meta["status"] == "complete" and meta["points"] == 6
    with (out / "summary.csv").open() as f:
        rows = list(csv.DictReader(f))
    assert {r["workload"] for r in rows} == {"layernorm_backward", "rowwise_quant", "layernorm_backward_stats"}
    assert all(float(r["dsmem_ms"]) > 0 and r["measured_cluster_size"] == "4" for r in rows)
    # the saved bundle can be re-scored offline
    again = spawn([sys.executable, "-m", "credit_b200.runner", "--rescore", out])
    assert again.returncode == 0 and json.loads(again.stdout)["points"] == 6


REFERENCE_BIN = ROOT / "oracle" / "_ref"
REFERENCE_WORKLOADS = ("layernorm_backward", "weighted_var_backward", "pearson_backward", "softmax_logits_backward",
                       "lars_momentum", "rowwise_quant")


@pytest.mark.parametrize("name", REFERENCE_WORKLOADS)
def test_beside_the_reference_binary(name, record_property):
    """The reference's own executable (built from its sources into oracle/_ref by oracle/Makefile,
    when those sources were at hand) and this project's, same flags, same GPU, at the reference's
    default cluster size 8 and its largest sweep width: both verify their results in-binary, both
    print the protocol `runner.parse_cuda_output` reads, and this project's cluster kernel is not
    slower than the reference's (measured 1.4x - 2x faster)."""
    ref = REFERENCE_BIN / name
    if not ref.exists():
        pytest.skip("oracle/_ref is not built here (needs the reference sources at build time)")
    flags = ["--csv", "--n-values", "65536", "--warmup", 5, "--iters", 20, "--cluster-size", 8]
    theirs = spawn([ref] + flags)
    ours = spawn([BIN / name] + flags)
    assert theirs.returncode == 0, theirs.stdout[-1500:] + theirs.stderr[-1500:]
    assert ours.returncode == 0, ours.stdout[-1500:] + ours.stderr[-1500:]
    (t,) = runner.parse_cuda_output(theirs.stdout)
    (o,) = runner.parse_cuda_output(ours.stdout)
    assert (t["cols"], t["rows"]) == (o["cols"], o["rows"])
    record_property("reference_cluster_ms", t["cluster_ms"])
    record_property("credit_b200_cluster_ms", o["cluster_ms"])
    print(f"{name}: reference block {t['block_ms']:.4f} cluster {t['cluster_ms']:.4f} ms (P={t['cluster_size']}); "
          f"credit_b200 block {o['block_ms']:.4f} cluster {o['cluster_ms']:.4f} ms (P={o['cluster_size']})")
    assert o["cluster_ms"] <= t["cluster_ms"] * 1.02
