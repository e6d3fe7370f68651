"""Builds the native library in-tree with nvcc for sm_100a.

The reference builds one executable per `.cu` with a Makefile
(`Makefile:33-40`, `nvcc -std=c++17 -O3 -arch=$(CUDA_ARCH)`); here every kernel
goes into one shared library, `credit_b200/lib/libcredit_b200.so`, plus thin
command-line front ends that link against it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
REPO_ROOT = PACKAGE_DIR.parent
CSRC = PACKAGE_DIR / "csrc"
LIB_DIR = PACKAGE_DIR / "lib"
BIN_DIR = PACKAGE_DIR / "bin"
LIB_PATH = LIB_DIR / "libcredit_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-std=c++17", "-O3", "-lineinfo", *ARCH_FLAGS]

# Translation units of the shared library (every other file in csrc/ is a header).
LIB_SOURCES = [
    "launch.cu",
    "tables_rmsnorm.cu",
    "tables_layernorm_fwd.cu",
    "tables_layernorm_bwd.cu",
    "tables_layernorm_bwd_f32.cu",
    "tables_layernorm_bwd_bf16.cu",
    "tables_row_reduce.cu",
    "ffn_kernels.cu",
    "tables_block_read.cu",
    "tables_row_ops.cu",
    "bench_entry.cu",
    "host_entry.cu",
    "tables_ws_rmsnorm.cu",
    "tables_ws_layernorm_fwd.cu",
    "tables_ws_layernorm_bwd.cu", "tables_ws_layernorm_bwd_dx.cu",
    "tables_ws_row_ops.cu",
    "comm_entry.cu", "peer_allreduce.cu",
]
OBJ_DIR = LIB_DIR / "obj"
# name of the executable -> (source, links against the shared library)
CLI_SOURCES: dict[str, tuple[str, bool]] = {
    "primitive_benchmark": ("primitive_benchmark.cu", False),
    "cluster_control": ("cluster_control.cu", False),
    "workload_bench": ("workload_bench.cu", True),
}
# workload_bench takes its workload from the name it is started under: it is
# installed once per workload, as the reference has one executable per workload.
WORKLOAD_BINARIES = ["layernorm_backward", "rmsnorm_forward", "row_reduce", "layernorm_forward",
                     "layernorm_backward_stats", "weighted_var_backward", "pearson_backward",
                     "softmax_logits_backward", "lars_momentum", "rowwise_quant"]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the native library cannot be built")
    return found


def _newest_source_mtime() -> float:
    paths = list(CSRC.glob("*")) + [REPO_ROOT / "include" / "credit_b200.h"]
    return max(p.stat().st_mtime for p in paths if p.is_file())


def _run(cmd: list[str], verbose: bool) -> str:
    result = subprocess.run(cmd, text=True, capture_output=True, check=False)
    if result.returncode != 0:
        raise RuntimeError(
            f"command failed ({result.returncode}): {' '.join(cmd)}\n{result.stdout}\n{result.stderr}"
        )
    if verbose:
        sys.stderr.write(result.stdout + result.stderr)
    return result.stdout + result.stderr


def _compile_object(source: str, verbose: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (Path(source).stem + ".o")
    cmd = [nvcc_path(), *COMMON_FLAGS, "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-c",
           str(CSRC / source), "-o", str(obj)]
    return obj, _run(cmd, verbose)


def build_library(force: bool = False, verbose: bool = False, ptxas_log: Path | None = None) -> Path:
    """Compiles libcredit_b200.so if it is missing or older than its sources. The
    translation units are compiled in parallel and linked into one shared library."""
    from concurrent.futures import ThreadPoolExecutor

    LIB_DIR.mkdir(parents=True, exist_ok=True)
    if not force and LIB_PATH.exists() and LIB_PATH.stat().st_mtime >= _newest_source_mtime():
        return LIB_PATH
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(len(LIB_SOURCES), os.cpu_count() or 1)) as pool:
        results = list(pool.map(lambda src: _compile_object(src, verbose), LIB_SOURCES))
    objects = [str(obj) for obj, _ in results]
    _run([nvcc_path(), *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *objects, "-ldl"], verbose)
    if ptxas_log is not None:
        ptxas_log.write_text("\n".join(log for _, log in results))
    return LIB_PATH


def build_cli(force: bool = False, verbose: bool = False) -> list[Path]:
    """Compiles the command-line front ends (they link against the library)."""
    BIN_DIR.mkdir(parents=True, exist_ok=True)
    build_library(force=force, verbose=verbose)
    built = []
    for name, (source, needs_lib) in CLI_SOURCES.items():
        out = BIN_DIR / name
        src = CSRC / source
        newest = max(_newest_source_mtime(), LIB_PATH.stat().st_mtime if needs_lib else 0.0)
        if not force and out.exists() and out.stat().st_mtime >= newest:
            built.append(out)
            continue
        cmd = [nvcc_path(), *COMMON_FLAGS, "-o", str(out), str(src)]
        if needs_lib:
            cmd += [f"-L{LIB_DIR}", "-lcredit_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib"]
        _run(cmd, verbose)
        built.append(out)
    generic = BIN_DIR / "workload_bench"
    for name in WORKLOAD_BINARIES:
        target = BIN_DIR / name
        if force or not target.exists() or target.stat().st_mtime < generic.stat().st_mtime:
            shutil.copy2(generic, target)
        built.append(target)
    return built


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_library(force=force, verbose=verbose)
    build_cli(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB_PATH)
