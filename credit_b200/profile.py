"""Parses the output of `primitive_benchmark` into a device profile.

Same labels, same keys and the same `DeviceProfile` construction as the reference
(`dsmem_eval/profile.py:27-126`), so text produced by either tool parses here; the
per-cluster-size lines that only this project's benchmark prints ("Cluster  8
mbarrier exchange : ...") land in `parsed["per_cluster"][8]`.
"""
from __future__ import annotations

import re
from dataclasses import asdict
from typing import Any

from .cost_model import B200Calibration, DeviceProfile

_FLOAT = r"([0-9]+(?:\.[0-9]+)?)"

# key -> (pattern, description); every pattern is anchored at a line start
_REQUIRED = {
    "clock_ghz": (rf"^Clock frequency:\s*{_FLOAT}\s+GHz", "clock frequency"),
    "l1_latency_cycles": (rf"^L1\s+read latency\s*:\s*{_FLOAT}\s+cycles", "L1 latency"),
    "l2_latency_cycles": (rf"^L2\s+read latency\s*:\s*{_FLOAT}\s+cycles", "L2 latency"),
    "dram_latency_cycles": (rf"^DRAM read latency\s*:\s*{_FLOAT}\s+cycles", "DRAM latency"),
    "l1_bytes_per_cycle_sm": (rf"^L1 cache bandwidth\s*:\s*{_FLOAT}\s+B/cycle/SM", "L1 bandwidth"),
    "l2_bytes_per_cycle": (rf"^L2 cache bandwidth\s*:\s*{_FLOAT}\s+B/cycle", "L2 bandwidth"),
    "dram_bandwidth_gbps": (rf"^Global memory bandwidth\s*:\s*{_FLOAT}\s+GB/s", "DRAM bandwidth"),
    "cluster_sync_cycles": (rf"^Cluster sync latency\s*:\s*{_FLOAT}\s+cycles/sync",
                            "cluster synchronization latency"),
    "local_smem_read_latency_cycles": (rf"^Local SMEM read latency\s*:\s*{_FLOAT}\s+cycles/load",
                                       "local SMEM latency"),
    "dsmem_read_latency_cycles": (rf"^DSMEM read latency\s*:\s*{_FLOAT}\s+cycles/load", "DSMEM read latency"),
    "local_smem_read_bytes_per_cycle_cta": (rf"^Local SMEM read throughput\s*:\s*{_FLOAT}\s+B/cycle/CTA",
                                            "local SMEM throughput"),
    "dsmem_read_bytes_per_cycle_cta": (rf"^DSMEM read throughput\s*:\s*{_FLOAT}\s+B/cycle/CTA",
                                       "DSMEM read throughput"),
    "local_smem_store_bytes_per_cycle_cta": (rf"^Local SMEM store throughput\s*:\s*{_FLOAT}\s+B/cycle/CTA",
                                             "local SMEM store throughput"),
    "dsmem_store_bytes_per_cycle_cta": (rf"^DSMEM store issue throughput\s*:\s*{_FLOAT}\s+B/cycle/CTA",
                                        "DSMEM store throughput"),
    "store_visibility_roundtrip_cycles": (rf"^Store visibility round trip\s*:\s*{_FLOAT}\s+cycles/roundtrip",
                                          "store visibility round trip"),
}

_PER_CLUSTER = {
    "sync_cycles": "sync latency",
    "barrier_exchange_cycles": "barrier exchange",
    "mbarrier_exchange_cycles": "mbarrier exchange",
    "dsmem_read_latency_cycles": "DSMEM read latency",
    "dsmem_read_bytes_per_cycle_cta": "DSMEM read throughput",
    "dsmem_store_bytes_per_cycle_cta": "DSMEM store throughput",
}


def _search(pattern: str, text: str, label: str) -> str:
    match = re.search(pattern, text, flags=re.MULTILINE)
    if match is None:
        raise RuntimeError(f"primitive benchmark did not report {label}")
    return match.group(1)


def parse_primitive_output(output: str) -> dict[str, Any]:
    parsed: dict[str, Any] = {
        "name": _search(r"^GPU Model:\s*(.+)$", output, "the GPU model").strip(),
        "sm_count": int(_search(r"^SM count:\s*(\d+)", output, "SM count")),
    }
    for key, (pattern, label) in _REQUIRED.items():
        parsed[key] = float(_search(pattern, output, label))
    per_cluster: dict[int, dict[str, float]] = {}
    for key, label in _PER_CLUSTER.items():
        for match in re.finditer(rf"^Cluster\s+(\d+)\s+{re.escape(label)}\s*:\s*{_FLOAT}", output, flags=re.MULTILINE):
            per_cluster.setdefault(int(match.group(1)), {})[key] = float(match.group(2))
    parsed["per_cluster"] = per_cluster
    parsed["bulk_copy_latency_cycles"] = {
        int(m.group(1)): float(m.group(2))
        for m in re.finditer(rf"^Bulk copy\s+(\d+) B latency\s*:\s*{_FLOAT}\s+cycles", output, flags=re.MULTILINE)
    }
    # DSMEM bulk copies (shared memory -> a peer CTA's shared memory): cluster size -> bytes ->
    # (cycles per step with one copy in flight, bytes per cycle and CTA with several in flight)
    dsmem_bulk: dict[int, dict[int, tuple[float, float]]] = {}
    for m in re.finditer(rf"^Cluster\s+(\d+)\s+DSMEM bulk\s+(\d+) B step\s*:\s*{_FLOAT}\s+cycles\s+\({_FLOAT} B/cycle/CTA",
                         output, flags=re.MULTILINE):
        dsmem_bulk.setdefault(int(m.group(1)), {})[int(m.group(2))] = (float(m.group(3)), float(m.group(4)))
    parsed["dsmem_bulk_copy"] = dsmem_bulk
    return parsed


def make_device_profile(parsed: dict[str, Any], properties: Any) -> DeviceProfile:
    """`properties` is anything with multi_processor_count, L2_cache_size and
    shared_memory_per_block_optin (torch's device properties, or a stand-in)."""
    clock_ghz = float(parsed["clock_ghz"])
    return DeviceProfile(
        name=str(parsed["name"]),
        sm_count=int(properties.multi_processor_count),
        clock_ghz=clock_ghz,
        hbm_bandwidth_gbps=float(parsed["dram_bandwidth_gbps"]),
        l2_capacity_bytes=int(properties.L2_cache_size),
        l2_bandwidth_gbps=float(parsed["l2_bytes_per_cycle"]) * clock_ghz,
        local_smem_bytes_per_cycle_cta=float(parsed["local_smem_read_bytes_per_cycle_cta"]),
        local_smem_store_bytes_per_cycle_cta=float(parsed["local_smem_store_bytes_per_cycle_cta"]),
        dsmem_store_bytes_per_cycle_cta=float(parsed["dsmem_store_bytes_per_cycle_cta"]),
        max_shared_bytes_per_cta=int(properties.shared_memory_per_block_optin),
    )


def measured_hbm_gbps(path: Any = None) -> float | None:
    """The copy ceiling of this machine's GPU from a MEASURED_PEAKS.json (key hbm_gbs) at `path`
    or at the repository root, if one exists."""
    import json
    from pathlib import Path
    candidate = Path(path) if path is not None else Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(candidate.read_text())["hbm_gbs"])
    except Exception:
        return None


def make_b200_calibration(parsed: dict[str, Any], hbm_gbps: float | None = None,
                          clock_ghz: float | None = None) -> B200Calibration:
    """Calibration of the row-period model from a parsed benchmark: the exchange cost per
    cluster size comes from the "mbarrier exchange" lines when they are present; the copy ceiling
    is the given one, else the machine's measured one (measured_hbm_gbps), else the default."""
    if hbm_gbps is None:
        hbm_gbps = measured_hbm_gbps()
    exchange = {p: v["mbarrier_exchange_cycles"] for p, v in parsed.get("per_cluster", {}).items()
                if "mbarrier_exchange_cycles" in v}
    if exchange:
        exchange.setdefault(1, min(exchange.values()) * 0.5)
    default = B200Calibration()
    return B200Calibration(
        clock_ghz=clock_ghz if clock_ghz is not None else default.clock_ghz,
        hbm_gbps=hbm_gbps if hbm_gbps is not None else default.hbm_gbps,
        exchange_cycles=exchange or None,
    )


def profile_as_dict(profile: DeviceProfile) -> dict[str, Any]:
    return asdict(profile)
