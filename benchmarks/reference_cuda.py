"""Time the REFERENCE's own CUDA GEMV on this GPU -- the second baseline of the sweep.

The reference ships no Blackwell-specific code: its CMake adds a plain ``sm_100`` cubin of its
SIMT kernels when the toolkit knows the architecture (``packages/dynquant-kernels/CMakeLists.txt:
153-165``, kernels ``csrc/gemv/gemv.cu:275-432`` and ``:444-555``).  ``oracle/build_ref.py``
compiles those sources where they lie into ``oracle/_ref/libdynquant_ref_cuda.so``; this script
loads that library -- in a process of its own, because it registers the ``dynquant::`` operator
namespace this package registers too -- and times ``torch.ops.dynquant.gemv`` with the sweep's
method: a CUDA graph of back-to-back calls over a ring of distinct weight tensors larger than
twice the L2, CUDA events around one replay.

    python benchmarks/reference_cuda.py '[{"rows": 4096, "in_features": 4096, "bits": 4, "group_size": 128, "m": 1}, ...]'

prints one JSON object per point: the point's keys plus ``reference_cuda_us`` and
``reference_cuda_gbps``.  The reference operator wants activations in the scales' dtype (bf16
for both here) and at most 8 rows; other points are skipped.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "oracle" / "_ref" / "libdynquant_ref_cuda.so"


def main() -> None:
    points = json.loads(sys.argv[1])
    launches = int(sys.argv[2]) if len(sys.argv) > 2 else 40
    if not LIB.exists():
        print(json.dumps({"unavailable": f"{LIB} is not built (python oracle/build_ref.py, needs the reference checkout)"}))
        return
    torch.ops.load_library(str(LIB))
    dev = torch.device("cuda")
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    for pt in points:
        rows, k, bits, group, m = pt["rows"], pt["in_features"], pt["bits"], pt["group_size"], pt["m"]
        if m > 8 or k % group:
            continue
        wpr, groups = k * bits // 32, k // group
        nbytes = rows * wpr * 4 + 2 * rows * groups * 2
        ring = max(1, min(64, -(-2 * l2 // nbytes)))
        gen = torch.Generator(device=dev).manual_seed(1)
        weights = []
        for _ in range(ring):
            packed = torch.randint(-(2**31), 2**31, (rows, wpr), dtype=torch.int32, device=dev, generator=gen)
            scales = (torch.rand(rows, groups, device=dev, generator=gen) * 0.015 + 0.005).to(torch.bfloat16)
            offsets = (-(1 << (bits - 1)) * scales.float()).to(torch.bfloat16)
            weights.append((packed, scales, offsets))
        x = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)

        def step(w):
            return torch.ops.dynquant.gemv(x, w[0], w[1], w[2], bits, group, k)

        for w in weights[: min(3, ring)]:
            step(w)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(launches):
                step(weights[i % ring])
        graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        seconds = start.elapsed_time(stop) / 1e3 / launches
        total = nbytes + m * k * 2 + m * rows * 2
        print(json.dumps({**pt, "reference_cuda_us": round(seconds * 1e6, 2),
                          "reference_cuda_gbps": round(total / seconds / 1e9, 1)}), flush=True)
        del weights, graph


if __name__ == "__main__":
    main()
