"""Host-side checks that need no GPU: the library builds, loads, and exports every
entry point the public header declares; the ctypes prototypes cover the same set."""
import ctypes
import re
from pathlib import Path

import pytest

from credit_b200 import _native

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "credit_b200.h"


def declared_functions() -> list[str]:
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(credit_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for required in ("credit_rmsnorm_forward", "credit_row_reduce", "credit_layernorm_forward",
                     "credit_layernorm_backward", "credit_layernorm_backward_stats",
                     "credit_query_device", "credit_last_error", "credit_plan"):
        assert required in names


def test_library_exports_every_declared_symbol(native_lib):
    for name in declared_functions():
        assert hasattr(native_lib, name), f"{name} is declared in the header but not exported"


def test_ctypes_prototypes_cover_the_header():
    assert sorted(_native.PROTOTYPES) == declared_functions()


def test_struct_sizes_match_the_header_layout():
    assert ctypes.sizeof(_native.LaunchOpts) == 8 * 4
    assert ctypes.sizeof(_native.DeviceInfo) == 256 + 11 * 4
    assert ctypes.sizeof(_native.PlanInfo) == 16 * 4 + 8
    fields = [n for n, _ in _native.LaunchOpts._fields_]
    header = HEADER.read_text()
    block = header[header.index("typedef struct credit_launch_opts"):header.index("} credit_launch_opts;")]
    assert re.findall(r"int (\w+);", block) == fields
    block = header[header.index("typedef struct credit_plan_info"):header.index("} credit_plan_info;")]
    assert re.findall(r"(?:int|size_t) (\w+);", block) == [n for n, _ in _native.PlanInfo._fields_]
    block = header[header.index("typedef struct credit_device_info"):header.index("} credit_device_info;")]
    assert re.findall(r"(?:int|char) (\w+)(?:\[256\])?;", block) == [n for n, _ in _native.DeviceInfo._fields_]


def test_make_opts_rejects_unknown_keys():
    with pytest.raises(ValueError):
        _native.make_opts({"cluster": 4})
    o = _native.make_opts({"cluster_size": 4, "stages": 2})
    assert o.cluster_size == 4 and o.stages == 2 and o.threads == 0


def test_last_error_is_a_string(native_lib):
    assert isinstance(_native.last_error(), str)
