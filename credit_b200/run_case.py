"""Runs one workload a few times on cuda:0 and checks the device status word.

The small driver behind profiler captures and quick timings:

    python -m credit_b200.run_case layernorm_backward_stats 1024 65536 \
        '{"cluster_size": 8, "threads": 512, "stages": 2}' 3
    python -m credit_b200.run_case ffn_forward 2048 4096 '{"hidden": 16384}' 3

Arguments: workload, rows, cols, launch options as JSON (optional), iterations
(optional, default 3). Prints one JSON line with the CUDA-event time per call.
Inputs are seeded draws with the distributions of the workload registry.
"""
from __future__ import annotations

import json
import sys

import torch

from . import _native as N
from . import launchers as L
from . import workloads as W


def main(argv: list[str]) -> int:
    if len(argv) < 3:
        print(__doc__)
        return 2
    name, rows, cols = argv[0], int(argv[1]), int(argv[2])
    opts = json.loads(argv[3]) if len(argv) > 3 else {}
    iters = int(argv[4]) if len(argv) > 4 else 3
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)

    if name == "ffn_forward":
        hidden = int(opts.pop("hidden", 4 * cols))
        x, w1, w2, gamma = W.make_ffn_inputs(rows, cols, dev, hidden=hidden)
        w1p, w2p = L.pack_ffn_weight(w1), L.pack_ffn_weight(w2)
        y = torch.empty_like(x)
        ws = torch.empty(L.ffn_workspace_bytes(rows, cols, hidden), dtype=torch.uint8, device=dev)

        def call():
            L.launch_ffn_forward((x, w1p, w2p, gamma), (y,), workspace=ws)
        work = W.ffn_flops(rows, cols, hidden)
        unit = "TFLOP/s"
    else:
        spec = W.WORKLOADS[name]
        cluster = int(opts.pop("cluster_size", 0))
        ins = spec.input_factory(rows, cols, dev)
        outs = L.allocate_outputs(name, ins)
        kw = {}
        if name == "layernorm_backward_stats":
            need = L.layernorm_backward_stats_workspace_bytes(rows, cols, spec.dtype)
            kw["workspace"] = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)

        def call():
            L.NATIVE_LAUNCHERS[name](ins, outs, cluster, dict(opts), **kw)
        work = W.algorithmic_bytes(name, rows, cols)
        unit = "GB/s"

    call()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        call()
    stop.record()
    stop.synchronize()
    ms = start.elapsed_time(stop) / iters
    status = N.device_status()
    rate = work / ms / (1e9 if unit == "TFLOP/s" else 1e6)
    print(json.dumps({"workload": name, "rows": rows, "cols": cols, "ms": round(ms, 5), unit: round(rate, 1),
                      "device_status": status}))
    return 0 if status == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main(sys.argv[1:]))
