"""MoE grouped GEMV: decode tokens/s and fraction of the HBM roofline (BASELINE config 4).

Qwen3-30B-A3B-shaped expert layer: 128 experts, top-8, hidden 2048, expert intermediate 768,
seeded widths, routing = top-8 of the softmax of seeded N(0,1) logits, 1..64 tokens per step.

    python -m dynquant_b200.moe_bench [--tokens 1,2,4,8,16,32,64] [--layers 6]
    python -m torch.distributed.run --nproc-per-node N ... -m dynquant_b200.moe_bench --ep

Single GPU: ``--layers`` distinct expert layers run back to back per step (their banks
together exceed L2, so expert weights come from HBM).  Algorithmic bytes per layer-step =
packed bytes of the DISTINCT activated experts (once each) + token activations + routing.
``--ep``: experts placed over the ranks, tokens exchanged by all-to-all
(:class:`dynquant_b200.sharded.ExpertParallelMoE`); every rank contributes tokens/world tokens.
Prints one JSON object per token count.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from . import ops
from .sweep import hbm_peak_gbs
from .workloads import qwen3_moe_layer, seeded_routing


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,2,4,8,16,32,64")
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--ep", action="store_true", help="expert-parallel over the torchrun ranks")
    ap.add_argument("--mode", default="all_to_all", choices=["all_to_all", "replicated"])
    ns = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if ns.ep:
        import torch.distributed as dist_mod

        dist = dist_mod
        import datetime

        # a short timeout: a rank that fails must end the others' next collective, not hang them
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    peak, kind = hbm_peak_gbs()
    widths = [(3, 4), (2, 3), (4, 2), (3, 3), (4, 4), (2, 4)]
    layers = [qwen3_moe_layer("cpu" if ns.ep else dev, seed=3030 + i, bits_gate_up=widths[i % 6][0],
                              bits_down=widths[i % 6][1]) for i in range(ns.layers)]
    if ns.ep:
        from .sharded import ExpertParallelMoE, expert_shard

        eps = [ExpertParallelMoE(expert_shard(l.gate_up, 2 * l.inter, l.num_experts, rank, world).to(dev),
                                 expert_shard(l.down, l.hidden, l.num_experts, rank, world).to(dev),
                                 num_experts=l.num_experts) for l in layers]
    for tokens in (int(t) for t in ns.tokens.split(",")):
        if ns.ep and (tokens % world or tokens // world == 0):
            continue
        t_local = tokens // world if ns.ep else tokens
        ids_all, w_all = seeded_routing(tokens, 128, 8, seed=99 + tokens)
        mine = slice(rank * t_local, (rank + 1) * t_local) if ns.ep else slice(0, tokens)
        ids, w = ids_all[mine].to(dev).contiguous(), w_all[mine].to(dev).contiguous()
        x = torch.randn(t_local, 2048, device=dev).to(torch.bfloat16)
        scratch = torch.empty(ops.moe_scratch_bytes(max(tokens, 1), 8, 2048, 768, 128, torch.bfloat16),
                              dtype=torch.uint8, device=dev)

        def step():
            for i in range(ns.layers):
                if ns.ep:
                    eps[i](x, ids, w, mode=ns.mode)
                else:
                    ops.moe_gemv(x, ids, w, layers[i].gate_up, layers[i].down, num_experts=128, scratch=scratch)

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        # Single GPU: replay a CUDA graph of the step, so that the time is the device's.  With
        # --ep the step runs eagerly: its NCCL exchanges are issued from Python, rank by rank,
        # and the time includes that host work.
        run, launch = step, "eager"
        if not ns.ep:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            graph.replay()
            torch.cuda.synchronize()
            run, launch = graph.replay, "cuda graph"
        if dist is not None:
            dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(ns.steps):
            run()
        stop.record()
        torch.cuda.synchronize()
        seconds = start.elapsed_time(stop) / 1e3 / ns.steps / ns.layers
        if dist is not None:
            t = torch.tensor([seconds], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            seconds = float(t.item())
        nbytes = sum(l.bytes_for(ids_all, tokens) for l in layers) / ns.layers
        if rank == 0:
            print(json.dumps({
                "workload": "qwen3-30b-a3b expert layer", "tokens": tokens, "n_gpus": world,
                "exchange": ns.mode if ns.ep else None, "launch": launch,
                "us_per_layer": round(seconds * 1e6, 2), "tokens_per_s_per_layer": round(tokens / seconds, 1),
                "activated_experts": int(torch.unique(ids_all).numel()),
                "algorithmic_mb_per_layer": round(nbytes / 1e6, 2), "gbps": round(nbytes / seconds / 1e9, 1),
                "pct_of_hbm_peak": round(100 * nbytes / seconds / 1e9 / (peak * world), 1),
                "peak": f"{peak} GB/s per GPU ({kind})",
            }), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
