#!/usr/bin/env python
"""Headline benchmark: packed mixed-precision decode GEMV on B200.

One "step" is one pass of the hot path over every packed linear module of the
synthetic Qwen-style 2B decode stack (28 layers, hidden 2048, intermediate 6144,
16 q / 8 kv heads of 128, seeded width map over {2,3,4,8} with a nominal mean of
3.25 bits, 8-bit lm_head of 248,320 rows) at M=1 with bf16 activations: 197
GEMV launches, 1.1 GB of packed weights, larger than L2 by an order of
magnitude, so every step re-reads its weights from HBM.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

prints ONE JSON line.  `value` is algorithmic GB/s with inputs resident in HBM;
`e2e` is the same metric through the public runner with the step's activations
copied in from pinned host memory and the logits copied back, inside the timed
region; `roofline` relates the dominant kernel to the measured HBM peak;
`cpu_baseline` times the reference's CPU path on a bounded sample of the same
workload on this machine's host cores.

Under torchrun (N > 1) every module is column-sharded over the ranks and the
pieces the next module needs are all-gathered over NCCL; value is whole-job.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "packed_gemv_hbm_gbps_m1"
UNIT = "GB/s"
WORKLOAD = "qwen2b-stack-3.25bit-m1 (BASELINE config 2: 28 layers + 8-bit lm_head, 197 GEMVs/step)"
FALLBACK_HBM_GBS = 6650.0
TRAFFIC_PER_STEP = 1_165_303_296  # dram bytes read + written by one step; see profiles/stack_qwen2b_m1_launch_list.md


def measured_peak() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    QUERY = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.file = None

    def __enter__(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL,
            )
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.file is None:
            return out
        self.file.flush()
        rows = [r.split(",") for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 8]
        os.unlink(self.file.name)
        sm, reasons = [], set()
        for r in rows:
            r = [c.strip() for c in r]
            try:
                sm.append(float(r[1]))
                out["sm_max_mhz"] = float(r[2])
            except ValueError:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6),
                              ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        if sm:
            # under load = the upper half of the samples (idle samples bracket the region)
            sm.sort()
            out["sm_mhz"] = statistics.median(sm[len(sm) // 2:])
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def cpu_baseline_sample(stack_modules, m: int, budget_modules: int = 56, repeat: int = 8) -> dict:
    """Time the reference CPU path on the first ``budget_modules`` modules of the stack: eight
    decoder layers (184 MB of packed weights, more than the host's last-level cache), eight
    passes -- about ten seconds of CPU work at the ~0.2 GB/s the reference's operator reaches."""
    sample = [(mod.weight.num_rows, mod.weight.in_features, mod.weight.bits) for mod in stack_modules[:budget_modules]]
    spec = {"modules": sample, "m": m, "repeat": repeat, "seed": 7}
    res = subprocess.run(
        [sys.executable, str(ROOT / "oracle" / "cpu_baseline.py"), json.dumps(spec)],
        capture_output=True, text=True, timeout=900,
    )
    if res.returncode != 0:
        return {"value": None, "unit": UNIT, "cores": None, "kind": "port", "sample": f"failed: {res.stderr[-200:]}"}
    out = json.loads(res.stdout.strip().splitlines()[-1])
    return {
        "value": round(out["gbps"], 4), "unit": UNIT, "cores": out["cores"], "kind": out["kind"],
        "sample": f"{out['modules']} GEMVs (first {budget_modules} modules of the stack x{repeat}, "
                  f"{out['bytes'] / 1e6:.1f} MB algorithmic) in {out['seconds']:.2f} s",
        "seconds": round(out["seconds"], 3),
    }


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def run_reference(args) -> None:
    """Reference arm: the reference's own CPU implementation of the path on the host cores."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from dynquant_b200.workloads import _decoder_layers, seeded_bit_map

    specs = _decoder_layers(28, 2048, 6144, 2048, 1024)
    names = [s[0] for s in specs]
    bit_map = seeded_bit_map(names, {2: 54, 3: 79, 4: 53, 8: 10}, 20260)
    sample = [(r, k, bit_map[n]) for (n, r, k, _) in specs[:7]]
    spec = {"modules": sample, "m": 1, "repeat": 1, "seed": 7}
    times, last = [], None
    for i in range(args.warmup + args.steps):
        res = subprocess.run(
            [sys.executable, str(ROOT / "oracle" / "cpu_baseline.py"), json.dumps(spec)],
            capture_output=True, text=True, timeout=900,
        )
        if res.returncode != 0:
            print(json.dumps({"impl": "reference", "unavailable": res.stderr.strip()[-200:]}))
            return
        last = json.loads(res.stdout.strip().splitlines()[-1])
        if i >= args.warmup:
            times.append(last["seconds"])
    sec = sum(times) / len(times)
    value = last["bytes"] / sec / 1e9
    sample_txt = "layer 0 of the stack (7 GEMVs, %.1f MB algorithmic) per step" % (last["bytes"] / 1e6)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "m": 1, "sample": sample_txt},
        "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": last["cores"], "kind": last["kind"],
                         "sample": sample_txt},
        "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def time_steps(fn, steps: int, warmup: int, sync, barrier):
    """W untimed steps, then exactly K steps between CUDA events on the current stream."""
    import torch

    for _ in range(warmup):
        fn()
    sync()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    sync()
    barrier()
    return start.elapsed_time(stop) / 1e3  # seconds


def run_ours(args) -> None:
    import torch

    rank, world, local = dist_env()
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        import datetime

        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=120))

    from dynquant_b200 import _lib
    from dynquant_b200.stack import StepRunner
    from dynquant_b200.workloads import qwen2b_stack

    _lib.load()
    m = args.m
    full = qwen2b_stack(device="cpu" if False else device, layers=args.layers)  # generated on the GPU
    if world > 1:
        from dynquant_b200.sharded import ShardedStepRunner

        use_graph = not args.no_graph
        runner = ShardedStepRunner(full, m, rank=rank, world=world, device=device,
                                   graph_mode=args.graph_mode if use_graph else None)
        step_fn = runner.run
        launches_per_step = runner.launches_per_step
    else:
        runner = StepRunner(full, m, device=device)
        use_graph = not args.no_graph
        if use_graph:
            runner.capture(args.graph_mode)
            step_fn = runner.replay
        else:
            step_fn = runner.run
            runner.count_launches()
        launches_per_step = runner.launches_per_step
    step_bytes = full.algorithmic_bytes(m)

    def sync():
        torch.cuda.synchronize(device)

    def barrier():
        if dist is not None:
            dist.barrier()

    with ClockSampler(local) as clocks:
        seconds = time_steps(step_fn, args.steps, args.warmup, sync, barrier)
        time.sleep(0.15)
    clock_summary = clocks.summary()
    if dist is not None:
        t = torch.tensor([seconds], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds = float(t.item())
    per_step = seconds / args.steps
    value = step_bytes / per_step / 1e9

    # ---- end to end: activations in from pinned host memory, logits back ----
    host_in = {k: v.cpu().pin_memory() for k, v in runner.inputs.items()}
    last_name = full.modules[-1].name
    logits_dev = runner.outputs[last_name]  # sharded runs: the gathered pieces, same bytes
    host_out = torch.empty_like(logits_dev, device="cpu").pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host_in.values())
    d2h = host_out.numel() * host_out.element_size()

    io_graph = world == 1 and use_graph and args.graph_mode in ("plan", "dataflow", "chain") and not args.e2e_eager_copies
    if io_graph:
        # the serving loop's form: pinned staging buffers, copies and kernels in one graph
        runner.capture_with_io(host_in, last_name, host_out, args.graph_mode)

    def e2e_step():
        if io_graph:
            runner.replay_with_io()
        else:
            for k, v in host_in.items():
                runner.inputs[k].copy_(v, non_blocking=True)
            step_fn()
            host_out.copy_(logits_dev, non_blocking=True)
        torch.cuda.current_stream(device).synchronize()

    for _ in range(args.warmup):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_seconds = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_seconds], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_seconds = float(t.item())
    e2e_value = step_bytes / (e2e_seconds / args.steps) / 1e9

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    # The second denominator: what a read-only stream and a copy reach on this GPU, now, through
    # this library's own launch path (the reference quotes against the same pair, measured in
    # its own session: commands/bench.py:95-120).  Outside the timed regions.
    probe = None
    if not args.no_probe:
        from dynquant_b200 import ops as _ops

        probe = _ops.achievable_bandwidth(nbytes=4 << 30, iters=10, device=device)
    launches = launches_per_step * args.steps
    avg_launch_s = seconds / launches
    bytes_per_launch = step_bytes / launches_per_step
    achieved = bytes_per_launch / avg_launch_s / 1e9 * (world if world > 1 else 1) / max(world, 1)
    # dram__bytes_read.sum + dram__bytes_write.sum of one step, from the ncu launch list of this
    # very command (profiles/stack_qwen2b_m1_launch_list.md), spread over the step's launches.
    traffic = (round(TRAFFIC_PER_STEP / launches_per_step)
               if (args.layers == 28 and m == 1 and world == 1) else None)
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(per_step * 1e3, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": WORKLOAD if args.layers == 28 else f"qwen2b-stack reduced to {args.layers} layers",
            "m": m, "activations": "bf16", "scales": "fp16", "group_size": 128,
            "weight_bytes": full.weight_bytes, "algorithmic_bytes_per_step": step_bytes,
            "l2": "working set (1.1 GB of weights per step) is larger than L2; no flush needed",
            "launch": (f"cuda graph of one step, {args.graph_mode} edges, programmatic dependent launch"
                       if use_graph else "dq_gemv_sequence per step"),
            "parallelism": ("single gpu" if world == 1 else
                            f"large layers ({', '.join(runner.sharded)}) column-sharded x{world} with an NCCL "
                            f"all-gather, small layers computed on every rank"),
            "peak": f"{peak} GB/s ({peak_kind})",
        },
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
            "frac": round(achieved / peak, 4), "traffic": traffic,
            "kernel": "gemv_mma_tile_kernel (decoder-block layers, fused shards) / gemv_mma_stream_kernel "
                      f"(lm_head); per-launch average over the {launches_per_step} launches of a step",
            "bytes_per_launch": round(bytes_per_launch), "avg_launch_us": round(avg_launch_s * 1e6, 3),
            "probe": (None if probe is None else {
                "read_gbs": round(probe["read_gbs"], 1), "copy_gbs": round(probe["copy_gbs"], 1),
                "bytes": probe["bytes"], "frac_of_read": round(achieved / probe["read_gbs"], 4),
                "kernels": "dq_probe_read / dq_probe_copy, 10 launches each, CUDA events"}),
        },
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "copies": "in the step's graph (pinned staging buffers)" if io_graph else "separate calls around the step"},
        "gpu_launches": launches,
        "clocks": clock_summary,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_sample(full.modules, m)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--m", type=int, default=1, help="activation rows (decode batch)")
    ap.add_argument("--layers", type=int, default=28, help="reduce the stack (profiling only)")
    ap.add_argument("--no-graph", action="store_true", help="launch with dq_gemv_sequence instead of a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-probe", action="store_true", help="skip the read/copy bandwidth probe")
    ap.add_argument("--e2e-eager-copies", action="store_true",
                    help="end-to-end arm: issue the host<->device copies as separate calls around the step's graph")
    ap.add_argument("--graph-mode", choices=["plan", "dataflow", "chain", "independent"], default="plan",
                    help="edges of the captured step: a decoder layer's data dependencies (default), "
                         "a strict chain, or none")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
