#!/usr/bin/env python
"""Headline benchmark: packed mixed-precision decode GEMV on B200.

One "step" is one pass of the hot path over every packed linear module of the
synthetic Qwen-style 2B decode stack (28 layers, hidden 2048, intermediate 6144,
16 q / 8 kv heads of 128, seeded width map over {2,3,4,8} with a nominal mean of
3.25 bits, 8-bit lm_head of 248,320 rows) at M=1 with bf16 activations: 197
GEMVs, 1.15 GB of packed weights -- larger than L2 by an order of magnitude, so
every step re-reads its weights from HBM.  The step replays from a CUDA graph:
by default one launch per stage of a decoder layer's data flow (the members of
a stage -- q/k/v, gate/up -- fused into one launch), ``--graph-mode plan`` for
the whole step as one persistent kernel (``dq_plan_*``).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

prints ONE JSON line.  ``value`` is algorithmic GB/s with inputs resident in HBM;
``e2e`` is the same metric through the public runner with the step's activations
copied in from pinned host memory and the logits copied back, inside the timed
region; ``roofline`` relates the kernel that dominates the step to the measured
HBM peak; ``cpu_baseline`` times the reference's CPU path on a bounded sample of
the same workload on this machine's host cores.  Two more blocks carry the rest
of the metric, measured in the same process after the headline region: ``moe``
(expert layer of BASELINE's fourth configuration: tokens/s, us per layer and
fraction of the roofline at 1, 8 and 64 tokens) and ``config3`` (the Qwen3-14B-
shaped linear set of the third configuration).

Under torchrun (N > 1) the modules whose per-rank slab is still large (the
lm_head) are column-sharded over the ranks and their outputs all-gathered by the
producing launch itself over peer memory (``--exchange fused``; ``peer``: the
library's exchange kernels, ``nccl``: NCCL calls); small modules are computed by
every rank; ``value`` is whole-job, and the line says whether the gathered
output equals the unsharded result.  The ``config3`` block shards every module
and the ``moe`` block places the experts over the ranks.
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
REFERENCE_THREADS = 16  # host threads of the reference arm and the cpu baseline, at every N


def measured_peak() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


# dram__bytes_read.sum + dram__bytes_write.sum of the 112 gemv_mma_tile_kernel launches of one
# step (638.2 MB), per launch, from an ncu launch list of the default command on a B200.
TILE_KERNEL_DRAM_BYTES_PER_LAUNCH = 5_698_000


EXCHANGE_WORDS = {
    "fused": "by the producing GEMV launch itself: stores into every rank's window over peer memory and a bounded "
             "wait, in the graph",
    "peer": "library exchange kernels over peer memory, in the graph",
    "nccl": "NCCL, issued after the graph",
    "none": "nothing to exchange",
    None: "nothing to exchange",
}


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
        self.skip = 0

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

    def rows_so_far(self) -> int:
        if self.file is None:
            return 0
        return sum(1 for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 8)

    def wait_for_first_sample(self, limit_s: float = 8.0) -> None:
        """nvidia-smi takes a while to start (longer with one per rank on an eight-GPU box): the
        timed region begins only once it is sampling."""
        end = time.time() + limit_s
        while self.proc is not None and self.rows_so_far() == 0 and time.time() < end:
            time.sleep(0.05)

    def mark_load_start(self) -> None:
        """Samples taken before this call are idle ones and are left out of the summary."""
        self.skip = self.rows_so_far()

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
        rows = rows[self.skip:]
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
            out["sm_mhz"] = statistics.median(sm)
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def run_cpu_sample(spec: dict) -> dict:
    """One run of the CPU timing script in a child process, with a fixed thread count: under
    ``torch.distributed.run`` the environment carries OMP_NUM_THREADS=1, which would make the
    reference arm slower at N > 1 than at N = 1."""
    threads = min(REFERENCE_THREADS, os.cpu_count() or 1)
    env = {**os.environ, "OMP_NUM_THREADS": str(threads), "MKL_NUM_THREADS": str(threads)}
    spec = {**spec, "threads": threads}
    res = subprocess.run([sys.executable, str(ROOT / "oracle" / "cpu_baseline.py"), json.dumps(spec)],
                         capture_output=True, text=True, timeout=900, env=env)
    if res.returncode != 0:
        raise RuntimeError(res.stderr.strip()[-300:])
    return json.loads(res.stdout.strip().splitlines()[-1])


def cpu_baseline_sample(stack_modules, m: int, budget_modules: int = 56, repeat: int = 8) -> dict:
    """Time the reference CPU path on the first ``budget_modules`` modules of the stack: eight
    decoder layers (184 MB of packed weights, more than the host's last-level cache), eight
    passes -- about ten seconds of CPU work at the ~0.2 GB/s the reference's operator reaches."""
    sample = [(mod.weight.num_rows, mod.weight.in_features, mod.weight.bits) for mod in stack_modules[:budget_modules]]
    try:
        out = run_cpu_sample({"modules": sample, "m": m, "repeat": repeat, "seed": 7})
    except (RuntimeError, subprocess.TimeoutExpired) as exc:
        return {"value": None, "unit": UNIT, "cores": None, "kind": "port", "sample": f"failed: {exc}"}
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
        try:
            last = run_cpu_sample(spec)
        except (RuntimeError, subprocess.TimeoutExpired) as exc:
            print(json.dumps({"impl": "reference", "unavailable": str(exc)[-200:]}))
            return
        if i >= args.warmup:
            times.append(last["seconds"])
    sec = sum(times) / len(times)
    value = last["bytes"] / sec / 1e9
    sample_txt = "layer 0 of the stack (7 GEMVs, %.1f MB algorithmic) per step" % (last["bytes"] / 1e6)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": WORKLOAD, "m": 1, "sample": sample_txt},
        "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": last["cores"], "kind": last["kind"],
                         "sample": sample_txt},
        "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def time_steps(fn, steps: int, warmup: int, sync, barrier, on_start=None):
    """W untimed steps, then exactly K steps between CUDA events on the current stream."""
    import torch

    for _ in range(warmup):
        fn()
    sync()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    if on_start is not None:
        on_start()
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    sync()
    barrier()
    return start.elapsed_time(stop) / 1e3  # seconds


def max_over_ranks(seconds: float, dist, device) -> float:
    if dist is None:
        return seconds
    import torch

    t = torch.tensor([seconds], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def capture_runner(runner, mode: str) -> str:
    """Capture a StepRunner in ``mode``; a stack the plan kernel cannot take falls back to the
    launch-per-stage graph (still this library's kernels).  Returns the mode in use."""
    if mode == "plan":
        try:
            runner.capture("plan")
            return "plan"
        except RuntimeError as exc:
            if "dq_gemv_sequence" not in str(exc):
                raise
            mode = "dataflow"
    runner.capture(mode)
    return mode


def full_sharded_names(full, world: int, shard_min_bytes: int = 32 << 20) -> list[str]:
    return [mod.name for mod in full.modules
            if mod.weight.num_rows % world == 0 and mod.weight.nbytes // world >= shard_min_bytes]


def config3_block(args, rank, world, device, dist, peak) -> dict:
    """BASELINE's third configuration: the Qwen3-14B-shaped linear set (40 layers, hidden 5120,
    intermediate 17408, seeded 3/4-bit map), every module column-sharded over the ranks (each
    rank generates and holds only its slab of rows), M = 1.  Under N > 1 every stage's output
    slabs are all-gathered right after the stage, before the next stage's launch."""
    import torch

    from dynquant_b200.stack import StepRunner
    from dynquant_b200.workloads import qwen14b_linear_set

    local = qwen14b_linear_set(device=device, shard=(rank, world))
    if world == 1:
        runner = StepRunner(local, 1, device=device)
        mode = capture_runner(runner, args.graph_mode)
        step = runner.replay
        exchange = None
    else:
        from dynquant_b200.sharded import ShardedStepRunner

        mode = "dataflow" if args.graph_mode == "plan" else args.graph_mode
        runner = ShardedStepRunner(local, 1, rank=rank, world=world, device=device, graph_mode=mode,
                                   exchange=args.exchange, presharded=True)
        step = runner.run
        exchange = runner.exchange

    def sync():
        torch.cuda.synchronize(device)

    def barrier():
        if dist is not None:
            dist.barrier()

    steps = max(5, args.steps // 3)
    seconds = max_over_ranks(time_steps(step, steps, 3, sync, barrier), dist, device) / steps
    if world > 1:
        runner.check()
    local_bytes = local.algorithmic_bytes(1)
    total_bytes = local_bytes * world
    return {
        "workload": "qwen3-14b-shaped linear set (BASELINE config 3: 40 layers x 7 modules, 3/4-bit, M=1)",
        "placement": ("single gpu" if world == 1 else
                      f"every module column-sharded x{world}; each stage's output slabs all-gathered right after the "
                      f"stage ({EXCHANGE_WORDS[exchange]})"),
        "exchanges_per_step": 0 if world == 1 else runner.gathers_per_step,
        "stages_exchanged_by_their_own_launch": 0 if world == 1 else runner.fused_stages,
        "launch": f"cuda graph, {mode}", "launches_per_step": runner.launches_per_step,
        "ms_per_step": round(seconds * 1e3, 4), "weight_bytes_per_gpu": local.weight_bytes,
        "gbps_aggregate": round(total_bytes / seconds / 1e9, 1),
        "gbps_per_gpu": round(local_bytes / seconds / 1e9, 1),
        "frac_of_hbm_peak_per_gpu": round(local_bytes / seconds / 1e9 / peak, 4),
    }


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
        import datetime

        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=120))

    from dynquant_b200 import _lib
    from dynquant_b200.stack import StepRunner
    from dynquant_b200.workloads import LinearStack, qwen2b_stack

    _lib.load()
    m = args.m
    full = qwen2b_stack(device=device, layers=args.layers)  # generated on the GPU, same on every rank
    use_graph = not args.no_graph
    sharded_matches = None
    if world > 1:
        from dynquant_b200.sharded import ShardedStepRunner

        runner = ShardedStepRunner(full, m, rank=rank, world=world, device=device,
                                   graph_mode=args.graph_mode if use_graph else None, exchange=args.exchange)
        step_fn = runner.run
        mode = runner.graph_mode
        local_bytes = runner.local_stack.algorithmic_bytes(m)
    else:
        runner = StepRunner(full, m, device=device)
        mode = None
        if use_graph:
            mode = capture_runner(runner, args.graph_mode)
            step_fn = runner.replay
        else:
            step_fn = runner.run
            runner.count_launches()
        local_bytes = full.algorithmic_bytes(m)
    launches_per_step = runner.launches_per_step
    step_bytes = full.algorithmic_bytes(m)

    def sync():
        torch.cuda.synchronize(device)

    def barrier():
        if dist is not None:
            dist.barrier()

    with ClockSampler(local) as clocks:
        clocks.wait_for_first_sample()
        seconds = time_steps(step_fn, args.steps, args.warmup, sync, barrier, on_start=clocks.mark_load_start)
        seconds = max_over_ranks(seconds, dist, device)
        # The timed region can be shorter than the sampling period: the same steps keep running,
        # untimed, for ~0.35 s (the same count on every rank) so that samples are taken under
        # this very load.
        for _ in range(max(1, int(0.35 / (seconds / args.steps)))):
            step_fn()
        sync()
        barrier()
    clock_summary = clocks.summary()
    per_step = seconds / args.steps
    value = step_bytes / per_step / 1e9
    if world == 1 and mode == "plan":
        runner.plan().check()  # no stage's bounded wait ran out during the timed steps
    if world > 1:
        runner.check()  # nor an exchange's

    # ---- sharded runs: the gathered output against the same module computed unsharded ----
    if world > 1 and runner.sharded:
        name = runner.sharded[-1]
        mod = next(mm for mm in full.modules if mm.name == name)
        single = StepRunner(LinearStack("check", full.hidden, full.intermediate, [mod], full.bit_map), m, device=device)
        single.inputs[mod.input].copy_(runner.inputs[mod.input])
        try:
            single.run_plan()
            single.plan().check()
        except RuntimeError:
            single.run()
        sync()
        same = torch.equal(single.outputs[name], runner.gathered(name))
        flag = torch.tensor([1 if same else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        sharded_matches = bool(flag.item())
        del single

    # ---- end to end: activations in from pinned host memory, logits back ----
    host_in = {k: v.cpu().pin_memory() for k, v in runner.inputs.items()}
    last_name = full.modules[-1].name
    # sharded runs: the gathered pieces, the same bytes (a view that may alternate between steps)
    logits = (lambda: runner.full_output(last_name)) if world > 1 and last_name in runner.sharded else (
        lambda: runner.outputs[last_name])
    logits_dev = logits()
    host_out = torch.empty(logits_dev.shape, dtype=logits_dev.dtype, device="cpu").pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host_in.values())
    d2h = host_out.numel() * host_out.element_size()

    io_graph = world == 1 and use_graph and mode in ("plan", "dataflow", "chain") and not args.e2e_eager_copies
    if io_graph:
        # the serving loop's form: pinned staging buffers, copies and kernels in one graph
        runner.capture_with_io(host_in, last_name, host_out, mode)

    def e2e_step():
        if io_graph:
            runner.replay_with_io()
        else:
            for k, v in host_in.items():
                runner.inputs[k].copy_(v, non_blocking=True)
            step_fn()
            host_out.copy_(logits(), non_blocking=True)
        torch.cuda.current_stream(device).synchronize()

    for _ in range(args.warmup):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_seconds = max_over_ranks(time.perf_counter() - t0, dist, device)
    e2e_value = step_bytes / (e2e_seconds / args.steps) / 1e9

    peak, peak_kind = measured_peak()

    # ---- the dominant kernel, on its own: bytes one launch moves / that launch's duration ----
    # One plan launch IS the step.  In the launch-per-stage modes the lm_head launch (45 % of the
    # bytes) is timed apart and the decoder-block launches get the rest of the step.
    launches = launches_per_step * args.steps
    if mode == "plan":
        kernel = "gemv_plan_kernel"
        kernel_bytes, kernel_seconds = local_bytes, per_step
        other = None
    else:
        head = full.modules[-1] if world == 1 else runner.local_stack.modules[-1]
        head_bytes = head.weight.nbytes + m * head.weight.in_features * 2 + m * head.weight.num_rows * 2
        hr = StepRunner(LinearStack("head", full.hidden, full.intermediate, [head], full.bit_map), m, device=device)
        hr.capture("chain")
        head_seconds = time_steps(hr.replay, 20, 3, sync, lambda: None) / 20
        kernel = "gemv_mma_tile_kernel"
        kernel_bytes = (local_bytes - head_bytes) / max(1, launches_per_step - 1)
        kernel_seconds = max(per_step - head_seconds, 1e-9) / max(1, launches_per_step - 1)
        other = {"kernel": "gemv_mma_stream_kernel (lm_head)", "bytes": head_bytes,
                 "us": round(head_seconds * 1e6, 2), "frac": round(head_bytes / head_seconds / 1e9 / peak, 4)}
        del hr
    achieved = kernel_bytes / kernel_seconds / 1e9
    # DRAM bytes per launch of that kernel: from a profiler's launch list of this very command
    # (1 GPU, the full stack, a launch per stage), not from this run -- and said so.
    traffic, traffic_source = None, "not measured in this run (needs a profiler pass)"
    if world == 1 and args.layers == 28 and m == 1 and kernel == "gemv_mma_tile_kernel":
        traffic = TILE_KERNEL_DRAM_BYTES_PER_LAUNCH
        traffic_source = ("separate ncu launch list of this command (dram read + write bytes of the 112 "
                          "tiled launches of one step / 112); a constant of that capture, not measured in this run")

    # The second denominator: what a read-only stream and a copy reach on this GPU, now, through
    # this library's own launch path (the reference quotes against the same pair, measured in
    # its own session: commands/bench.py:95-120).  Outside the timed regions.
    probe = None
    if not args.no_probe and rank == 0:
        from dynquant_b200 import ops as _ops

        probe = _ops.achievable_bandwidth(nbytes=4 << 30, iters=10, device=device)

    # ---- the rest of the metric: expert layer (config 4) and the 14B linear set (config 3) ----
    extras = {}
    parallelism = ("single gpu" if world == 1 else
                   f"large layers ({', '.join(full_sharded_names(full, world))}) column-sharded x{world}, their outputs "
                   f"all-gathered ({EXCHANGE_WORDS[args.exchange]}); "
                   f"small layers computed on every rank")
    weight_bytes = full.weight_bytes
    cpu_modules = [(mod.weight.num_rows, mod.weight.in_features, mod.weight.bits) for mod in full.modules[:56]]
    if not args.no_extras and args.layers == 28:
        del runner, step_fn, full, host_in, host_out, logits_dev, logits
        torch.cuda.empty_cache()
        sys.path.insert(0, str(ROOT / "benchmarks"))
        import moe_bench

        tokens = [t for t in (1, 8, 64) if world == 1 or (t % world == 0)]
        extras["moe"] = {
            "metric": "moe_decode_tokens_per_s", "n_gpus": world,
            "placement": "single gpu" if world == 1 else (
                f"experts placed over {world} ranks; tokens gathered and partial sums reduce-scattered by the "
                "library's kernels over peer memory, the layer in one cuda graph"),
            "points": moe_bench.measure(tokens, layers=6, steps=20, rank=rank, world=world, device=device, dist=dist),
        }
        torch.cuda.empty_cache()
        extras["config3"] = config3_block(args, rank, world, device, dist, peak)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(per_step * 1e3, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "workload": WORKLOAD if args.layers == 28 else f"qwen2b-stack reduced to {args.layers} layers",
            "m": m, "activations": "bf16", "scales": "fp16", "group_size": 128,
            "weight_bytes": weight_bytes, "algorithmic_bytes_per_step": step_bytes,
            "l2": "working set (1.1 GB of weights per step) is larger than L2; no flush needed",
            "launch": (f"cuda graph of one step: {mode}" if use_graph else "dq_gemv_sequence per step"),
            "parallelism": parallelism,
            "peak": f"{peak} GB/s ({peak_kind})",
        },
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
            "frac": round(achieved / peak, 4),
            "kernel": kernel, "bytes_per_launch": round(kernel_bytes), "launch_us": round(kernel_seconds * 1e6, 3),
            "per_gpu": world > 1,
            "traffic": traffic, "traffic_source": traffic_source,
            "step_average": {"bytes_per_launch": round(local_bytes / launches_per_step),
                             "launch_us": round(per_step / launches_per_step * 1e6, 3),
                             "frac": round(local_bytes / per_step / 1e9 / peak, 4)},
            "other_kernel": other,
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
    if sharded_matches is not None:
        line["sharded_matches"] = sharded_matches
    line.update(extras)
    if world == 1 and not args.no_cpu_baseline:
        try:
            out = run_cpu_sample({"modules": cpu_modules, "m": m, "repeat": 8, "seed": 7})
            line["cpu_baseline"] = {
                "value": round(out["gbps"], 4), "unit": UNIT, "cores": out["cores"], "kind": out["kind"],
                "sample": f"{out['modules']} GEMVs (first {len(cpu_modules)} modules of the stack x8, "
                          f"{out['bytes'] / 1e6:.1f} MB algorithmic) in {out['seconds']:.2f} s",
                "seconds": round(out["seconds"], 3),
            }
        except (RuntimeError, subprocess.TimeoutExpired) as exc:
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": None, "kind": "port", "sample": f"failed: {exc}"}
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
    ap.add_argument("--no-extras", action="store_true", help="skip the moe and config3 blocks")
    ap.add_argument("--exchange", choices=["fused", "peer", "nccl"], default="fused",
                    help="N > 1: a sharded stage's output is exchanged by the GEMV launch itself (stores into the peers' "
                         "windows), by the library's exchange kernels over peer memory (both in the graph), or by NCCL calls")
    ap.add_argument("--e2e-eager-copies", action="store_true",
                    help="end-to-end arm: issue the host<->device copies as separate calls around the step's graph")
    ap.add_argument("--graph-mode", choices=["plan", "dataflow", "chain", "independent"], default="dataflow",
                    help="the captured step: a launch per stage with a decoder layer's data dependencies (default, "
                         "the fastest measured), one whole-step plan kernel, a strict chain of launches, or "
                         "launches with no edges")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
