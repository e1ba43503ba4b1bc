"""One column-sharded decode step, exchange by exchange (BASELINE config 3 on N GPUs).

Every module of the Qwen3-14B-shaped linear set is split into row slabs over the ranks and each
stage's output is all-gathered.  The same step is timed with every exchange the library offers,
and once with no exchange at all (every rank's local kernels only: what the exchanges add is
the difference):

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/sharded_step.py
        [--layers 40] [--steps 30] [--modes fused,peer,nccl,local] [--m 1]

``fused``: the stage's GEMV launch stores its rows into every rank's window and waits for the
others (``dq_gemv_stage_push``).  ``peer``: the library's exchange kernels between the stages.
``nccl``: one NCCL all-gather per stage, issued eagerly after the graph of local kernels.
``local``: no exchange.  CUDA events, max over ranks; rank 0 prints one JSON object per mode.
"""

from __future__ import annotations

import argparse
import datetime
import json
import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--modes", default="fused,peer,nccl,local")
    ns = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import torch.distributed as dist

    # a short timeout: a rank that fails must end the others' next collective, not hang them
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    from dynquant_b200.sharded import ShardedStepRunner
    from dynquant_b200.stack import StepRunner
    from dynquant_b200.workloads import qwen14b_linear_set

    stack = qwen14b_linear_set(device=dev, layers=ns.layers, shard=(rank, world))
    nbytes = stack.algorithmic_bytes(ns.m)
    for mode in ns.modes.split(","):
        if mode == "local":
            runner = StepRunner(stack, ns.m, device=dev)
            runner.capture("dataflow")
            step, check, fused, launches = runner.replay, (lambda: None), 0, runner.launches_per_step
        else:
            runner = ShardedStepRunner(stack, ns.m, rank=rank, world=world, device=dev, exchange=mode, presharded=True)
            step, check, fused, launches = runner.run, runner.check, runner.fused_stages, runner.launches_per_step
        for _ in range(3):
            step()
        torch.cuda.synchronize(dev)
        dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(ns.steps):
            step()
        stop.record()
        torch.cuda.synchronize(dev)
        check()
        t = torch.tensor([start.elapsed_time(stop) / 1e3 / ns.steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds = float(t.item())
        stages = len(stack.stages())
        if rank == 0:
            print(json.dumps({
                "workload": f"qwen3-14b-shaped linear set, {ns.layers} layers, m={ns.m}, every module column-sharded x{world}",
                "exchange": mode, "n_gpus": world, "stages": stages, "launches_per_step": launches,
                "stages_exchanged_by_their_own_launch": fused,
                "ms_per_step": round(seconds * 1e3, 4), "us_per_stage": round(seconds * 1e6 / stages, 2),
                "gbps_per_gpu": round(nbytes / seconds / 1e9, 1), "gbps_aggregate": round(nbytes * world / seconds / 1e9, 1),
            }), flush=True)
        del runner, step, check
        torch.cuda.empty_cache()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
