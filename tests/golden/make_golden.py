"""Generates tests/golden/reference_workloads.npz by running the REFERENCE's own
eager PyTorch functions (dsmem_eval/workloads.py) on small seeded inputs.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

Seeds follow the reference's convention torch.manual_seed(1234 + cols)
(dsmem_eval/runner.py:358); inputs come from the reference's own input factories.
The inputs are stored next to the outputs so the check does not depend on the RNG
of the torch version that replays it.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

SHAPES = [(3, 96), (2, 1000)]


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref_root = Path(sys.argv[1])
    sys.path.insert(0, str(ref_root))
    from dsmem_eval.workloads import WORKLOADS  # type: ignore

    arrays: dict[str, np.ndarray] = {}
    for name, spec in WORKLOADS.items():
        for rows, cols in SHAPES:
            torch.manual_seed(1234 + cols)
            inputs = spec.input_factory(rows, cols, torch.device("cpu"))
            with torch.no_grad():
                outputs = spec.torch_function(*inputs)
            if not isinstance(outputs, tuple):
                outputs = (outputs,)
            key = f"{name}/{rows}x{cols}"
            for i, t in enumerate(inputs):
                arrays[f"{key}/in{i}"] = t.numpy()
            for i, t in enumerate(outputs):
                arrays[f"{key}/out{i}"] = t.numpy()
        arrays[f"{name}/atol"] = np.float64(spec.atol)
        arrays[f"{name}/rtol"] = np.float64(spec.rtol)
    out = Path(__file__).resolve().parent / "reference_workloads.npz"
    np.savez_compressed(out, **arrays)
    print(f"wrote {out} ({out.stat().st_size} bytes, {len(arrays)} arrays)")


if __name__ == "__main__":
    main()
