"""ctypes binding of `libcredit_b200.so` (the C ABI in `include/credit_b200.h`).

There is no CPU fallback: if the library has not been built, or a call fails,
an exception is raised. The reference has no such binding -- its pipeline spawns
executables (`dsmem_eval/runner.py:280-310`) -- so this module is the stub a
maintainer would add to load the native backend in-process.
"""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, Structure, c_char, c_char_p, c_float, c_int, c_int64, c_size_t,
                    c_void_p)
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libcredit_b200.so"

CREDIT_OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_UNSUPPORTED = -2
ERR_CUDA = -3
ERR_WORKSPACE = -4
ERR_DEVICE_STATUS = -5

F32 = 0
BF16 = 1
COMM_ID_BYTES = 128      # credit_comm_get_unique_id
PEER_HANDLE_BYTES = 64   # credit_peer_group_create

VARIANT_AUTO, VARIANT_BLOCK_READ, VARIANT_BLOCK_SMEM, VARIANT_CLUSTER_SMEM = 0, 1, 2, 3
LOAD_AUTO, LOAD_TMA, LOAD_LDG = 0, 1, 2
SCHEDULE_AUTO, SCHEDULE_ROW_PER_CLUSTER, SCHEDULE_PERSISTENT = 0, 1, 2
FLAG_NO_REGISTER_PATH = 1

WL_RMSNORM_FORWARD = 0
WL_ROW_REDUCE = 1
WL_LAYERNORM_FORWARD = 2
WL_LAYERNORM_BACKWARD = 3
WL_LAYERNORM_BACKWARD_STATS = 4
WL_WEIGHTED_VAR_BACKWARD = 5
WL_PEARSON_BACKWARD = 6
WL_SOFTMAX_LOGITS_BACKWARD = 7
WL_LARS_MOMENTUM = 8
WL_ROWWISE_QUANT = 9


class CreditError(RuntimeError):
    """A call into the native library returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"credit_b200 error {code}: {message}")
        self.code = code
        self.message = message


class UnsupportedShape(CreditError):
    """The shape does not fit the requested variant (the reference's "n/a")."""


class LaunchOpts(Structure):
    _fields_ = [
        ("cluster_size", c_int),
        ("variant", c_int),
        ("stages", c_int),
        ("threads", c_int),
        ("schedule", c_int),
        ("load_path", c_int),
        ("chunk_bytes", c_int),
        ("flags", c_int),
    ]


class DeviceInfo(Structure):
    _fields_ = [
        ("name", c_char * 256),
        ("sm_major", c_int),
        ("sm_minor", c_int),
        ("sm_count", c_int),
        ("cluster_launch", c_int),
        ("max_cluster_size", c_int),
        ("max_dynamic_smem_per_block", c_int),
        ("smem_per_sm", c_int),
        ("l2_bytes", c_int),
        ("clock_khz", c_int),
        ("mem_clock_khz", c_int),
        ("mem_bus_bits", c_int),
    ]


class PlanInfo(Structure):
    _fields_ = [
        ("cluster_size", c_int),
        ("variant", c_int),
        ("stages", c_int),
        ("threads", c_int),
        ("schedule", c_int),
        ("load_path", c_int),
        ("aligned", c_int),
        ("slice_elems", c_int),
        ("chunk_elems", c_int),
        ("vectors_per_thread", c_int),
        ("full_tiles", c_int),
        ("num_clusters", c_int),
        ("grid_ctas", c_int),
        ("smem_bytes", c_int),
        ("kernel_launches", c_int),
        ("workspace_bytes", c_size_t),
    ]

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name, _ in self._fields_}


_OPTS_P = POINTER(LaunchOpts)

# name -> (restype, argtypes); the single source for binding and for the
# "library exports everything the header declares" test.
PROTOTYPES: dict[str, tuple] = {
    "credit_last_error": (c_char_p, []),
    "credit_query_device": (c_int, [c_int, POINTER(DeviceInfo)]),
    "credit_device_status": (c_int, [POINTER(c_int), c_int]),
    "credit_plan": (c_int, [c_int, c_int64, c_int64, c_int, _OPTS_P, POINTER(PlanInfo)]),
    "credit_rmsnorm_forward": (
        c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, _OPTS_P, c_void_p]),
    "credit_row_reduce": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, _OPTS_P, c_void_p]),
    "credit_layernorm_forward": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                c_float, c_int, _OPTS_P, c_void_p]),
    "credit_layernorm_backward": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, _OPTS_P,
                c_void_p]),
    "credit_layernorm_backward_stats_workspace_bytes": (
        c_size_t, [c_int64, c_int64, c_int, _OPTS_P]),
    "credit_layernorm_backward_stats": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                c_int64, c_int64, c_int, _OPTS_P, c_void_p, c_size_t, c_void_p]),
    "credit_row_op": (
        c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                _OPTS_P, c_void_p]),
    "credit_bench": (c_int, [c_char_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, POINTER(ctypes.c_double)]),
    "credit_ffn_pack_weight": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "credit_ffn_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "credit_ffn_forward": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float,
                c_void_p, c_size_t, c_void_p]),
    "credit_layernorm_backward_stats_static_capacity": (c_size_t, []),
    "credit_layernorm_backward_stats_static": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                c_int64, c_int64, c_int, _OPTS_P, c_void_p]),
    "credit_row_reduce_host_scratch_bytes": (c_size_t, [c_int64, c_int64]),
    "credit_row_reduce_host": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, _OPTS_P, c_void_p,
                c_size_t, c_void_p]),
    "credit_rmsnorm_forward_host_scratch_bytes": (c_size_t, [c_int64, c_int64, c_int]),
    "credit_rmsnorm_forward_host": (
        c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, _OPTS_P, c_void_p, c_size_t,
                c_void_p]),
    "credit_layernorm_forward_host_scratch_bytes": (c_size_t, [c_int64, c_int64, c_int]),
    "credit_layernorm_forward_host": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int,
                _OPTS_P, c_void_p, c_size_t, c_void_p]),
    "credit_layernorm_backward_stats_host_scratch_bytes": (c_size_t, [c_int64, c_int64, c_int, _OPTS_P]),
    "credit_layernorm_backward_stats_host": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                c_int, _OPTS_P, c_void_p, c_size_t, c_void_p]),
    "credit_comm_get_unique_id": (c_int, [c_void_p]),
    "credit_comm_init_rank": (c_int, [POINTER(c_void_p), c_int, c_int, c_void_p]),
    "credit_comm_destroy": (c_int, [c_void_p]),
    "credit_layernorm_bwd_allreduce": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "credit_peer_group_create": (c_int, [POINTER(c_void_p), c_int, c_int, c_int64, c_void_p]),
    "credit_peer_group_connect": (c_int, [c_void_p, c_void_p]),
    "credit_peer_group_destroy": (c_int, [c_void_p]),
    "credit_peer_group_status": (c_int, [c_void_p]),
    "credit_layernorm_bwd_allreduce_peer": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "credit_ffn_forward_host_scratch_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "credit_ffn_forward_host": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p,
                c_size_t, c_void_p]),
}

_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Loads the library once; raises if it was never built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m credit_b200.build` "
            "(there is no CPU fallback)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().credit_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code == CREDIT_OK:
        return
    message = last_error()
    if code == ERR_UNSUPPORTED:
        raise UnsupportedShape(code, message)
    raise CreditError(code, message)


def make_opts(opts: "LaunchOpts | dict | None") -> "LaunchOpts | None":
    if opts is None or isinstance(opts, LaunchOpts):
        return opts
    known = {name for name, _ in LaunchOpts._fields_}
    unknown = set(opts) - known
    if unknown:
        raise ValueError(f"unknown launch options: {sorted(unknown)}")
    return LaunchOpts(**opts)


def opts_ref(opts: "LaunchOpts | dict | None"):
    o = make_opts(opts)
    return None if o is None else ctypes.byref(o)


def query_device(device: int = -1) -> DeviceInfo:
    info = DeviceInfo()
    check(load().credit_query_device(device, ctypes.byref(info)))
    return info


def device_status(reset: bool = True) -> int:
    """Synchronises and returns the device status word (0 = healthy)."""
    word = c_int(0)
    code = load().credit_device_status(ctypes.byref(word), 1 if reset else 0)
    if code not in (CREDIT_OK, ERR_DEVICE_STATUS):
        check(code)
    return word.value


def plan(workload: int, rows: int, cols: int, dtype: int, opts=None) -> PlanInfo:
    info = PlanInfo()
    check(load().credit_plan(workload, rows, cols, dtype, opts_ref(opts), ctypes.byref(info)))
    return info
