"""Old dispatch against new over the linear layers of real models, kernel by kernel.

Needs a tuning build (``python -m dynquant_b200.build --tuning``): the environment switches
``DQ_B200_ROWS_SMALL_M=0`` and ``DQ_B200_STREAM_SLICED=0`` (read by such a build only) take the
many-rows kernel below nine activation rows and the sliced streaming kernel out of the dispatch,
which is then the tiled / streaming kernels alone.  Every point is timed both ways -- CUDA events
around one CUDA graph over a ring of distinct weight tensors larger than twice the L2, so the
packed bytes come from HBM -- and the two outputs are compared.  One JSON object per
(shape, width): ``m<M>_old`` / ``m<M>_new`` = [us per call, kernel, largest relative difference
to the old output]; a last line counts the points that kept their kernel, got faster, got slower.

    python benchmarks/dispatch_regression.py [--group 64] [--m 1,4,8] [--shape ROWSxK ...]
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from dynquant_b200 import ops  # noqa: E402
from dynquant_b200.workloads import random_quant_tensor  # noqa: E402

# q/k/v, o, gate/up and down projections of hidden sizes 1536..8192
SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (1024, 4096), (3584, 3584), (512, 3584), (18944, 3584),
          (3584, 18944), (1536, 1536), (8960, 1536), (1536, 8960), (5120, 13824), (13824, 5120), (8192, 8192),
          (1024, 8192), (28672, 8192), (8192, 28672), (3072, 8192), (8192, 3072), (2048, 16384), (16384, 2048),
          (8192, 29568), (6144, 4096), (4608, 3584), (2560, 9728), (9728, 2560)]
SWITCHES = ("DQ_B200_ROWS_SMALL_M", "DQ_B200_STREAM_SLICED")


def timed(fn, ring, reps: int = 3) -> float:
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for q in ring[:2]:
            fn(q)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for q in ring:
                fn(q)
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1000 / len(ring))
    return best


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", action="append", help="ROWSxK; repeatable (default: 26 shapes of real models)")
    ap.add_argument("--bits", default="2,3,4,8")
    ap.add_argument("--group", type=int, default=128)
    ap.add_argument("--m", default="1,4,8")
    args = ap.parse_args()
    stamp = Path(__file__).resolve().parent.parent / "dynquant_b200" / "lib" / "obj" / "build_kind.txt"
    if not stamp.exists() or stamp.read_text().strip() != "tuning":
        print("note: not a tuning build -- the switches are ignored and both arms run the full dispatch "
              "(python -m dynquant_b200.build --tuning)", file=sys.stderr)
    shapes = [tuple(int(v) for v in s.split("x")) for s in args.shape] if args.shape else SHAPES
    rows_m = [int(v) for v in args.m.split(",")]
    same = better = worse = 0
    for rows, k in shapes:
        for bits in (int(b) for b in args.bits.split(",")):
            nbytes = rows * k * bits // 8
            n = max(2, min(24, (300 << 20) // nbytes + 1)) if nbytes < (150 << 20) else 3
            gen = torch.Generator(device="cuda").manual_seed(bits)
            ring = [random_quant_tensor(rows, k, bits, group_size=args.group, meta_dtype=torch.float16, device="cuda", generator=gen)
                    for _ in range(n)]
            rec = {"shape": [rows, k], "bits": bits, "group": args.group}
            for m in rows_m:
                x = torch.randn(m, k, device="cuda").to(torch.bfloat16)

                def fn(q):
                    return ops.gemv(x, q.packed, q.scales, q.offsets, bits, args.group, k, out_dtype=torch.float32)

                ref = None
                for label, env in (("old", {s: "0" for s in SWITCHES}), ("new", {})):
                    for s in SWITCHES:
                        os.environ.pop(s, None)
                    os.environ.update(env)
                    out = fn(ring[0])
                    torch.cuda.synchronize()
                    name = ops.last_kernel()
                    ref = out if ref is None else ref
                    err = float((out - ref).abs().max() / ref.abs().max())
                    rec[f"m{m}_{label}"] = [round(timed(fn, ring), 1), name, f"{err:.0e}"]
                old, new = rec[f"m{m}_old"], rec[f"m{m}_new"]
                if old[1] == new[1]:
                    same += 1
                elif new[0] > 1.03 * old[0]:
                    worse += 1
                else:
                    better += 1
            print(json.dumps(rec), flush=True)
            del ring
    print(json.dumps({"kept_their_kernel": same, "changed_not_slower": better, "changed_slower": worse}))


if __name__ == "__main__":
    main()
