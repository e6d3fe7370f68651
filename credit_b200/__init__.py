"""credit_b200: sm_100a wide-row cluster/DSMEM kernels behind a C ABI.

`credit_b200.launchers.NATIVE_LAUNCHERS` is the in-process launcher table,
`credit_b200.workloads.WORKLOADS` the workload registry. Every kernel lives in
`lib/libcredit_b200.so`; nothing here computes on the CPU.
"""
from . import _native  # noqa: F401
from .workloads import WORKLOADS, WorkloadSpec, algorithmic_bytes  # noqa: F401

__all__ = ["WORKLOADS", "WorkloadSpec", "algorithmic_bytes"]
