"""Cluster-size cost model.

Two models live here.

`estimate` is the reference's profitability model ("effective-bandwidth-overlap-v2",
`dsmem_eval/cost_model.py:62-141`) with the same inputs, outputs and arithmetic, so
result bundles stay comparable: predicted gain = re-read traffic saved - control
overhead - local replay - store residual - DSMEM stores, with the device constants
taken from `DeviceProfile`.

`predict_cluster_ms` is the B200 recalibration that the headline target asks for
(predict WHICH cluster size is fastest, not only whether clusters pay off). On
B200 the register-resident kernels are bound neither by the re-read the reference
model counts nor by DSMEM store bandwidth; what was measured is

    time(P) = smooth_max( HBM time of the compulsory bytes,
                          rows / resident_clusters(P) * row_period(P) )

where a cluster finishes one row every `row_period` = fixed latency chain (ring
wait, shared-memory reads, shuffle trees, mbarrier exchange, stores: about 1.4 us
for the first reduction of a row at 1.9 GHz) + a per-element term, and `resident_clusters(P)` is
what the driver's occupancy query returns for the kernel (GPC packing makes it far
from sm_count / P: 15 clusters of 8 CTAs at one CTA per SM on a 148-SM part).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Protocol


class WorkloadModelSpec(Protocol):
    rows: int
    modeled_bytes_per_element: float
    reread_bytes_per_element: float
    staged_bytes_per_element: int
    partial_count: int


MODEL_VERSION = "effective-bandwidth-overlap-v2"
B200_MODEL_VERSION = "b200-row-period-v1"


@dataclass(frozen=True)
class DeviceProfile:
    name: str
    sm_count: int
    clock_ghz: float
    hbm_bandwidth_gbps: float
    l2_capacity_bytes: int
    l2_bandwidth_gbps: float
    local_smem_bytes_per_cycle_cta: float
    local_smem_store_bytes_per_cycle_cta: float
    dsmem_store_bytes_per_cycle_cta: float
    max_shared_bytes_per_cta: int


@dataclass(frozen=True)
class ModelEstimate:
    effective_bandwidth_gbps: float
    saved_reread_ms: float
    control_overhead_ms: float
    local_replay_ms: float
    local_store_residual_ms: float
    dsmem_store_ms: float
    predicted_delta_ms: float
    predicted_profitable: bool

    @property
    def saved_hbm_ms(self) -> float:
        return self.saved_reread_ms

    @property
    def local_staging_ms(self) -> float:
        return self.local_replay_ms + self.local_store_residual_ms


def shared_bytes_per_cta(spec: WorkloadModelSpec, cols: int, cluster_size: int) -> int:
    return math.ceil(cols / cluster_size) * spec.staged_bytes_per_element


def estimate(spec: WorkloadModelSpec, cols: int, cluster_size: int, control_overhead_ms: float,
             profile: DeviceProfile, baseline_ms: float, rows: int | None = None) -> ModelEstimate:
    """The reference model, term by term (cost_model.py:62-141)."""
    n_rows = spec.rows if rows is None else rows
    if not math.isfinite(baseline_ms) or baseline_ms <= 0.0:
        raise ValueError("baseline_ms must be finite and positive")
    if spec.modeled_bytes_per_element <= 0.0:
        raise ValueError("modeled_bytes_per_element must be positive")
    cycles_to_ms = 1.0 / (profile.clock_ghz * 1.0e6)

    baseline_bytes = n_rows * cols * spec.modeled_bytes_per_element
    effective_gbps = baseline_bytes / (baseline_ms * 1.0e6)
    saved_ms = baseline_ms * spec.reread_bytes_per_element / spec.modeled_bytes_per_element

    resident = max(profile.sm_count // cluster_size, 1)
    waves = math.ceil(n_rows / resident)
    slice_bytes = shared_bytes_per_cta(spec, cols, cluster_size)

    dsmem_ms = waves * (4.0 * (cluster_size - 1) * spec.partial_count
                        / profile.dsmem_store_bytes_per_cycle_cta) * cycles_to_ms
    replay_ms = waves * slice_bytes / profile.local_smem_bytes_per_cycle_cta * cycles_to_ms
    source_bytes_per_cycle_cta = effective_gbps / (profile.clock_ghz * profile.sm_count)
    residual_cycles = slice_bytes * max(
        1.0 / profile.local_smem_store_bytes_per_cycle_cta - 1.0 / source_bytes_per_cycle_cta, 0.0)
    residual_ms = waves * residual_cycles * cycles_to_ms
    control_ms = max(control_overhead_ms, 0.0)
    delta = saved_ms - control_ms - replay_ms - residual_ms - dsmem_ms
    return ModelEstimate(effective_gbps, saved_ms, control_ms, replay_ms, residual_ms, dsmem_ms, delta,
                         delta > 0.0)


# ---------------------------------------------------------------------------
# B200 recalibration
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class B200Calibration:
    """Constants measured on B200 (the output of primitive_benchmark and the cluster-size
    sweeps); cycles are SM cycles at `clock_ghz`."""
    clock_ghz: float = 1.93                    # SM clock under these memory-bound kernels
    hbm_gbps: float = 6538.6                   # copy ceiling
    chain_cycles_per_stage: float = 1600.0     # first reduction of a row: ring wait, LDS, shuffle
                                               # trees, push, wait, stores
    chain_cycles_next_stage: float = 200.0     # every further dependent reduction of the row
    chain_cycles_per_warp: float = 20.0        # per stage: the CTA-local collection grows with its warps
    exchange_cycles: dict | None = None        # st.async + mbarrier all-to-all, per cluster size
    cycles_per_element_per_thread: float = 4.0   # issue cost of one row element in one thread
    one_shot_cycles: float = 6000.0            # cluster launch + barrier set-up + first load, per row,
                                               # when every cluster handles a single row
    overlap_exponent: float = 2.0              # time = (hbm^k + latency^k)^(1/k)
    generic_path_efficiency: float = 0.5       # slices too large for registers run on the shared-memory
                                               # re-read kernels: about half of the copy ceiling
    cta_launch_ns: float = 4.8                 # streaming kernels: CTA launch throughput of the device
    launch_base_us: float = 3.0                # fixed cost of a launch
    streaming_ctas_to_saturate: int = 320      # CTAs of the streaming reduction that fill HBM
    # warp-specialised pipeline (8 output warps): a row costs a cluster the larger of its CTAs'
    # share of the HBM bandwidth and the output warps' issue time
    ws_sm_gbps_cap: float = 58.0               # most one SM pulls through bulk copies (7.0 TB/s on 120 SMs)
    ws_fixed_cycles: float = 550.0             # per row and CTA, whatever the slice length
    ws_p16_penalty: float = 1.15               # clusters of 16 ran this much slower than the terms say
    ws_cycles_per_element_fwd: float = 28.0    # per row element a thread owns, forward kernels
    ws_cycles_per_element_bwd: float = 40.0    # LayerNorm backward with column sums
    ws_load_latency_us: float = 1.5            # a ring stage's request lands after about this long
    ws_cycles_per_element_bwd_dx: float = 36.0   # LayerNorm backward, dx only (two staged inputs)
    ws_cycles_per_element_per_array: float = 12.0   # reference-sweep workloads, per staged or written array
    ws_short_ring_penalty: float = 1.12        # fewer than five stages: the passes run one row apart
    ws_fill_rows: float = 3.0                  # ring fill, rows between the passes, the last cluster's extra row

    def exchange(self, cluster_size: int) -> float:
        table = self.exchange_cycles or {1: 150.0, 2: 315.0, 4: 322.0, 8: 351.0, 16: 420.0}
        return table.get(cluster_size, 420.0)


@dataclass(frozen=True)
class ClusterPrediction:
    cluster_size: int
    hbm_ms: float
    rows_per_cluster: int
    row_period_us: float
    predicted_ms: float


def predict_cluster_ms(rows: int, cols: int, cluster_size: int, resident_clusters: int, threads: int,
                       algorithmic_bytes: float, reduction_stages: int, persistent: bool = True,
                       cal: B200Calibration = B200Calibration(), register_path: bool = True) -> ClusterPrediction:
    """Predicted time of one call of a cluster kernel.
    resident_clusters: clusters of this shape that are co-resident (credit_plan's num_clusters for a
    persistent launch); threads: threads per CTA; register_path: the slice fits the register-resident
    kernels (credit_plan's vectors_per_thread > 0), otherwise the shared-memory re-read kernels run."""
    if min(rows, cols, cluster_size, resident_clusters, threads) <= 0:
        raise ValueError("all sizes must be positive")
    hbm_ms = algorithmic_bytes / (cal.hbm_gbps * 1.0e6)
    if not register_path:
        rows_per_cluster = math.ceil(rows / resident_clusters)
        return ClusterPrediction(cluster_size, hbm_ms, rows_per_cluster, 0.0, hbm_ms / cal.generic_path_efficiency)
    elems_per_thread = math.ceil(cols / cluster_size / threads)
    chain = (cal.chain_cycles_per_stage + (reduction_stages - 1) * cal.chain_cycles_next_stage +
             reduction_stages * (cal.chain_cycles_per_warp * (threads // 32) + cal.exchange(cluster_size)))
    period_cycles = chain + elems_per_thread * cal.cycles_per_element_per_thread
    if not persistent:
        period_cycles += cal.one_shot_cycles
    rows_per_cluster = math.ceil(rows / resident_clusters)
    row_period_us = period_cycles / (cal.clock_ghz * 1.0e3)
    latency_ms = rows_per_cluster * row_period_us * 1.0e-3
    # neither bound is reached exactly: the two overlap imperfectly (a cubic mean stays within a
    # few per cent of max() when one term dominates)
    k = cal.overlap_exponent
    predicted = (hbm_ms ** k + latency_ms ** k) ** (1.0 / k)
    return ClusterPrediction(cluster_size, hbm_ms, rows_per_cluster, row_period_us, predicted)


def predict_ws_ms(rows: int, cols: int, cluster_size: int, resident_clusters: int, threads: int,
                  elem_bytes: int, arrays_in: int, arrays_out: float, stages: int, backward: bool = False,
                  row_op: bool = False, cal: B200Calibration = B200Calibration()) -> ClusterPrediction:
    """Predicted time of one call of a warp-specialised kernel (threads 352 or 608 per CTA), the
    formula of the library's planner (launch.cu: predicted_ws_ms): the SMs the co-resident clusters
    cover share the copy ceiling, one SM pulls at most `ws_sm_gbps_cap`, and the output warps need
    a fixed number of cycles per row plus a number per row element a thread owns.
    arrays_in / arrays_out: arrays of the element type staged / written per row (0.25 for int8
    output of fp32 input)."""
    if min(rows, cols, cluster_size, resident_clusters, threads - 96) <= 0:
        raise ValueError("all sizes must be positive")
    slice_elems = -(-math.ceil(cols / cluster_size) // 64) * 64
    bytes_per_cta_row = (arrays_in + arrays_out) * slice_elems * elem_bytes
    sms = resident_clusters * cluster_size
    per_sm_gbps = min(cal.hbm_gbps / sms, cal.ws_sm_gbps_cap)
    hbm_us = bytes_per_cta_row / (per_sm_gbps * 1.0e3)
    elems = math.ceil(slice_elems / (threads - 96))
    per_elem = (cal.ws_cycles_per_element_bwd if backward else
                cal.ws_cycles_per_element_per_array * (arrays_in + arrays_out) if row_op else
                cal.ws_cycles_per_element_bwd_dx if arrays_in == 2 else
                cal.ws_cycles_per_element_fwd)
    issue_us = (cal.ws_fixed_cycles + per_elem * elems) / (cal.clock_ghz * 1.0e3)
    in_flight = max(1, stages - (3 if stages >= 5 else 2))   # ring stages that are loads on their way
    row_us = max(hbm_us, issue_us, cal.ws_load_latency_us / in_flight)
    row_us *= cal.ws_short_ring_penalty if stages < 5 else 1.0
    if cluster_size >= 16:
        row_us *= cal.ws_p16_penalty
    rows_per_cluster = math.ceil(rows / resident_clusters)
    predicted = row_us * (rows_per_cluster + cal.ws_fill_rows) * 1.0e-3
    hbm_ms = (arrays_in + arrays_out) * rows * cols * elem_bytes / (cal.hbm_gbps * 1.0e6)
    return ClusterPrediction(cluster_size, hbm_ms, rows_per_cluster, row_us, predicted)


def predict_streaming_ms(rows: int, cluster_size: int, algorithmic_bytes: float,
                         cal: B200Calibration = B200Calibration()) -> ClusterPrediction:
    """Predicted time of the streaming row reduction (nothing staged, one cluster per row):
    HBM time, stretched when rows x P CTAs are too few to keep HBM busy, or the time the device
    needs to launch that many CTAs, whichever is longer."""
    if min(rows, cluster_size) <= 0:
        raise ValueError("all sizes must be positive")
    hbm_ms = algorithmic_bytes / (cal.hbm_gbps * 1.0e6)
    ctas = rows * cluster_size
    fill = min(1.0, ctas / cal.streaming_ctas_to_saturate)
    launch_ms = ctas * cal.cta_launch_ns * 1.0e-6
    predicted = max(hbm_ms / fill, launch_ms) + cal.launch_base_us * 1.0e-3
    return ClusterPrediction(cluster_size, hbm_ms, 1, 0.0, predicted)


def best_cluster_size(predictions: list[ClusterPrediction], tie: float = 0.01) -> int:
    """Cluster size with the lowest predicted time; predictions within `tie` (1 %) of the lowest
    count as equal and the smallest cluster among them wins (it is the easiest to place)."""
    if not predictions:
        raise ValueError("no predictions")
    lowest = min(p.predicted_ms for p in predictions)
    return min(p.cluster_size for p in predictions if p.predicted_ms <= lowest * (1.0 + tie))


# ---------------------------------------------------------------------------
# The planner's rule for the warp-specialised kernels (launch.cu: plan_static), restated so that
# a host can know the launch without a GPU. Calibrated on a B200 sweep of cluster size x ring
# depth: small clusters cover more SMs and spread a row's fixed costs over longer slices, a ring
# of three stages costs 5 - 20 %, clusters of 16 are never worth it where 8 fits.
# ---------------------------------------------------------------------------
WS_CONTROL_BYTES = 22528          # control block at the start of a CTA's dynamic shared memory
WS_OUTPUT_THREADS = 256           # 8 output warps (threads = 352)
_WS_WANTED_STAGES = {"lars_momentum": 6, "weighted_var_backward": 3, "softmax_logits_backward": 3, "rowwise_quant": 3}
_WS_ROW_OPS = ("weighted_var_backward", "pearson_backward", "softmax_logits_backward", "lars_momentum", "rowwise_quant")


def ws_plan_rule(workload: str, cols: int, elem_bytes: int, arrays_in: int, column_sums: bool = False,
                 max_smem: int = 232448, max_cluster: int = 16) -> tuple[int, int] | None:
    """(cluster size, ring stages) the library launches for a 16-byte aligned row of `cols` elements
    when the caller leaves both to it, or None where no warp-specialised plan fits (the library
    then falls back to its other kernels). `arrays_in`: arrays staged per row; `column_sums`:
    LayerNorm backward with dgamma/dbeta (half the elements per thread). fp32 RMSNorm is not
    planned here: the library keeps its lock-step kernel for it."""
    if min(cols, elem_bytes, arrays_in) <= 0:
        raise ValueError("all sizes must be positive")
    row_op = workload in _WS_ROW_OPS
    max_slice = (1 << 30) if row_op else WS_OUTPUT_THREADS * (32 if column_sums else 64)

    def slice_elems(p: int) -> int:
        return -(-(-(-cols // p)) // 64) * 64

    def stage_bytes(p: int) -> int:
        return arrays_in * slice_elems(p) * elem_bytes

    def fits(p: int, stages: int) -> bool:
        return slice_elems(p) <= max_slice and WS_CONTROL_BYTES + stages * stage_bytes(p) <= max_smem

    sizes = [p for p in (1, 2, 4, 8, 16) if p <= max_cluster]
    wanted = _WS_WANTED_STAGES.get(workload, 4)
    with3 = next((p for p in sizes if fits(p, 3)), 0)
    with_wanted = next((p for p in sizes if fits(p, wanted)), 0)
    cluster = with_wanted or with3
    if cluster == 16 and 0 < with3 <= 8:
        cluster = with3
    if cluster == 0:
        return None
    per_stage = stage_bytes(cluster)

    def most(limit: int) -> int:
        return min(8, (limit - WS_CONTROL_BYTES) // per_stage)

    if row_op:
        stages = 6
    else:
        half = (max_smem - 2048) // 2
        stages = most(half) if most(half) >= 6 else most(max_smem)
    while stages > 3 and WS_CONTROL_BYTES + stages * per_stage > max_smem:
        stages -= 1
    return cluster, stages
