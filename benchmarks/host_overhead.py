"""Host time per packed-GEMV call, route by route.

The reference's decode step is host-bound: 20-45 us of Python and dispatch per packed module
around single-digit-microsecond kernels (experiments/four_point/RESULTS.md:884-892).  This
script measures what a caller of this library pays per call on a matrix small enough that the
kernel is negligible (256 x 256, 4-bit): wall time of N calls issued back to back, divided by N,
with the stream drained only at the end (so the figure is issue cost, not kernel time).

    python benchmarks/host_overhead.py [--calls 5000]

Routes: the C ABI through ctypes (``ops.gemv``), ``torch.ops.dynquant.gemv`` with the Python
backend and with the compiled C++ backend (each in a child process: the choice is made at
import), ``quantized_matmul`` on a QuantTensor, a ``DynQuantLinear`` module call, and one
``dq_gemv_sequence`` call for 100 such modules (per module).  Prints one JSON object.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def measure(calls: int) -> dict:
    import torch

    import dynquant_b200
    from dynquant_b200 import ops
    from dynquant_b200.runtime import DynQuantLinear
    from dynquant_b200.stack import StepRunner
    from dynquant_b200.workloads import LinearStack, Module, random_quant_tensor

    dev = torch.device("cuda")
    qt = random_quant_tensor(256, 256, 4, device=dev)
    x = torch.randn(1, 256, device=dev).to(torch.bfloat16)
    layer = DynQuantLinear(qt)

    def timed(fn) -> float:
        for _ in range(200):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(calls):
            fn()
        dt = time.perf_counter() - t0
        torch.cuda.synchronize()
        return dt / calls * 1e6

    out = {"torch_ops_backend": ops.torch_ops_backend()}
    args = (x, qt.packed, qt.scales, qt.offsets, 4, 128, 256)
    out["ops.gemv (ctypes)"] = round(timed(lambda: ops.gemv(*args)), 2)
    out["torch.ops.dynquant.gemv"] = round(timed(lambda: torch.ops.dynquant.gemv(*args)), 2)
    out["quantized_matmul"] = round(timed(lambda: dynquant_b200.quantized_matmul(x, qt)), 2)
    out["DynQuantLinear.__call__"] = round(timed(lambda: layer(x)), 2)
    stack = LinearStack("host", 256, 256, [Module(f"m{i}", qt, "hidden") for i in range(100)], {})
    runner = StepRunner(stack, 1, device=dev)
    out["dq_gemv_sequence per module (100 modules per call)"] = round(timed(runner.run) / 100, 3)
    runner.capture("dataflow")
    out["cuda graph replay per module (100 modules per graph)"] = round(timed(runner.replay) / 100, 3)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--calls", type=int, default=5000)
    ap.add_argument("--child", action="store_true")
    ns = ap.parse_args()
    if ns.child:
        print(json.dumps(measure(ns.calls)))
        return
    result = {"unit": "us of host time per call", "calls": ns.calls}
    for label, shim in (("c++ backend", "1"), ("python backend", "0")):
        res = subprocess.run([sys.executable, __file__, "--child", "--calls", str(ns.calls)], capture_output=True,
                             text=True, env={**os.environ, "DQ_B200_TORCH_SHIM": shim})
        if res.returncode != 0:
            result[label] = {"failed": res.stderr.strip()[-300:]}
        else:
            result[label] = json.loads(res.stdout.strip().splitlines()[-1])
    print(json.dumps(result, indent=1))


if __name__ == "__main__":
    main()
