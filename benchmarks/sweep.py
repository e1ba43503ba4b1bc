"""Width / shape sweep of the packed GEMV: achieved HBM GB/s and % of the roofline per point.

The counterpart of the reference's ``benchmarks/gemv_bandwidth.py`` for this library, and
BASELINE config 5: widths {2,3,4,8} x group {64,128} x Mistral-7B shapes x M {1,4,16} plus
odd-N tails.  Every point runs over a ring of distinct weight tensors whose total size
exceeds twice the L2 (so the bytes really come from HBM) and is timed with CUDA events;
M above the operator's row limit of 8 is issued as several GEMV launches up to 64 rows, and
through the dequant + dense path beyond, as in the reference.

    python benchmarks/sweep.py                      # the full config-5 grid
    python benchmarks/sweep.py --shape 131072x2048 --bits 8 --m 1 --launches 4 --ring 1
                                                       # one point, few launches (for ncu)
    python benchmarks/sweep.py --op dequant --shape 32768x4096 --group 128
                                                       # the dequant operator instead (write-bound)

Prints one JSON object per point.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from dynquant_b200 import ops  # noqa: E402
from dynquant_b200.workloads import random_quant_tensor  # noqa: E402


def hbm_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return 6650.0, "fallback"


def check_block(x: torch.Tensor, qt, out: torch.Tensor, rows_checked: int = 256) -> float:
    """Largest error of the LAST ``rows_checked`` output rows (the ragged tail included) against
    plain fp32 torch arithmetic on the dequantized rows, relative to the block's largest value.
    A timed number for a wrong result would be worthless; the parity tests proper are in tests/."""
    lo = max(0, qt.num_rows - rows_checked)
    dense = ops.dequantize(qt.rows(lo, qt.num_rows)).float()  # [rows_checked, K]
    want = x.float() @ dense.t()
    got = out[:, lo:].float()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def run_point(rows: int, k: int, bits: int, group: int, m: int, *, launches: int, ring: int | None,
              device="cuda") -> dict:
    probe = random_quant_tensor(rows, k, bits, group_size=group, device=device)
    l2 = torch.cuda.get_device_properties(device).L2_cache_size
    if ring is None:
        ring = max(1, min(64, -(-2 * l2 // probe.nbytes)))
    weights = [probe] + [random_quant_tensor(rows, k, bits, group_size=group, device=device) for _ in range(ring - 1)]
    x = torch.randn(m, k, device=device).to(torch.bfloat16)

    def step(qt):
        return ops.quantized_matmul(x, qt)

    for qt in weights[: min(3, ring)]:
        out = step(qt)
    kernel = ops.last_kernel()
    torch.cuda.synchronize()
    # the output is rounded once to bf16 (2^-8 relative), the fp32 sums differ in their last bits
    err = check_block(x, weights[min(3, ring) - 1], out)
    if not err <= 1e-2:
        raise SystemExit(f"{rows}x{k} bits={bits} group={group} m={m}: result differs from fp32 torch arithmetic ({err:.3e})")
    # one CUDA graph of `launches` back-to-back calls over the ring: device time only, no Python
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
    nbytes = probe.nbytes + m * k * 2 + m * rows * 2
    peak, kind = hbm_peak_gbs()
    gbs = nbytes / seconds / 1e9
    return {
        "rows": rows, "in_features": k, "bits": bits, "group_size": group, "m": m,
        "path": ("gemv" if m <= ops.gemv_max_rows() else
                 "dequant+dense" if m > ops.GEMV_CHUNKED_MAX_ROWS else
                 "many-rows kernel" if kernel == "gemv_rows_kernel" else "row chunks"),
        "kernel": kernel,
        "us_per_call": round(seconds * 1e6, 2), "gbps": round(gbs, 1),
        "pct_of_hbm_peak": round(100 * gbs / peak, 1), "peak": f"{peak} GB/s ({kind})",
        "ring": ring, "ring_bytes": probe.nbytes * ring, "launches": launches, "max_err_vs_fp32_torch": float(f"{err:.2e}"),
    }


def run_dequant_point(rows: int, k: int, bits: int, group: int, *, launches: int, device="cuda") -> dict:
    """Dense reconstruction of one packed tensor: bytes = packed + metadata read, dense written."""
    qt = random_quant_tensor(rows, k, bits, group_size=group, device=device)
    out = ops.dequantize(qt)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(launches):
            out = ops.dequantize(qt)
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    stop.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(stop) / 1e3 / launches
    nbytes = qt.nbytes + out.numel() * out.element_size()
    peak, kind = hbm_peak_gbs()
    return {
        "op": "dequant", "rows": rows, "in_features": k, "bits": bits, "group_size": group,
        "us_per_call": round(seconds * 1e6, 2), "gbps": round(nbytes / seconds / 1e9, 1),
        "pct_of_hbm_peak": round(100 * nbytes / seconds / 1e9 / peak, 1), "peak": f"{peak} GB/s ({kind})",
        "bytes": nbytes, "launches": launches,
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemv", choices=["gemv", "dequant"])
    ap.add_argument("--shape", action="append", help="ROWSxK; repeatable (default: the config-5 shapes)")
    ap.add_argument("--bits", default="2,3,4,8")
    ap.add_argument("--group", default="64,128")
    ap.add_argument("--m", default="1,4,16")
    ap.add_argument("--launches", type=int, default=50)
    ap.add_argument("--ring", type=int, default=None, help="distinct weight tensors (default: > 2x L2)")
    ap.add_argument("--no-reference", action="store_true",
                    help="skip the second baseline (the reference's own CUDA kernels, timed by a child process)")
    ns = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the sweep needs a CUDA device: this library has no CPU path")
    shapes = ns.shape or ["14336x4096", "4096x14336", "4096x4096", "4097x4096"]
    results = []
    for shape in shapes:
        rows, k = (int(v) for v in shape.lower().split("x"))
        for bits in (int(b) for b in ns.bits.split(",")):
            for group in (int(g) for g in ns.group.split(",")):
                if ns.op == "dequant":
                    print(json.dumps(run_dequant_point(rows, k, bits, group, launches=ns.launches)), flush=True)
                    continue
                for m in (int(v) for v in ns.m.split(",")):
                    point = run_point(rows, k, bits, group, m, launches=ns.launches, ring=ns.ring)
                    if ns.no_reference:
                        print(json.dumps(point), flush=True)
                    results.append(point)
    if ns.op == "dequant" or ns.no_reference:
        return
    # second baseline: the reference's own CUDA kernels, compiled for sm_100, on this GPU -- timed
    # by a child process (its library registers the same operator namespace as this package)
    reference = reference_cuda_points(results, ns.launches)
    peak, _ = hbm_peak_gbs()
    for point in results:
        ref = reference.get(point_key(point))
        if ref is not None:
            point["reference_cuda_us"] = ref["reference_cuda_us"]
            point["reference_cuda_pct_of_hbm_peak"] = round(100 * ref["reference_cuda_gbps"] / peak, 1)
            point["speedup_vs_reference_cuda"] = round(ref["reference_cuda_us"] / point["us_per_call"], 2)
        print(json.dumps(point), flush=True)


def point_key(p: dict) -> tuple:
    return (p["rows"], p["in_features"], p["bits"], p["group_size"], p["m"])


def reference_cuda_points(results: list[dict], launches: int) -> dict:
    import subprocess

    spec = [{k: p[k] for k in ("rows", "in_features", "bits", "group_size", "m")} for p in results]
    script = Path(__file__).resolve().parent / "reference_cuda.py"
    try:
        res = subprocess.run([sys.executable, str(script), json.dumps(spec), str(launches)], capture_output=True,
                             text=True, timeout=3600)
    except subprocess.TimeoutExpired:
        return {}
    out = {}
    for line in res.stdout.splitlines():
        try:
            row = json.loads(line)
        except ValueError:
            continue
        if "reference_cuda_us" in row:
            out[point_key(row)] = row
    return out


if __name__ == "__main__":
    main()
