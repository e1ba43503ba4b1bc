"""MoE grouped GEMV: decode tokens/s and fraction of the HBM roofline (BASELINE config 4).

Qwen3-30B-A3B-shaped expert layer: 128 experts, top-8, hidden 2048, expert intermediate 768,
seeded widths, routing = top-8 of the softmax of seeded N(0,1) logits, 1..64 tokens per step.

    python benchmarks/moe_bench.py [--tokens 1,2,4,8,16,32,64] [--layers 6]
    python -m torch.distributed.run --nproc-per-node N ... benchmarks/moe_bench.py --ep

Single GPU: ``--layers`` distinct expert layers run back to back per step (their banks
together exceed L2, so expert weights come from HBM).  Algorithmic bytes per layer-step =
packed bytes of the DISTINCT activated experts (once each) + token activations + routing.
``--ep``: experts placed over the ranks, tokens exchanged by all-to-all
(:class:`dynquant_b200.sharded.ExpertParallelMoE`); every rank contributes tokens/world tokens.
Prints one JSON object per token count.  ``bench.py`` calls :func:`measure` for its ``moe`` block.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from dynquant_b200 import ops  # noqa: E402
from dynquant_b200.workloads import qwen3_moe_layer, seeded_routing  # noqa: E402

WIDTHS = [(3, 4), (2, 3), (4, 2), (3, 3), (4, 4), (2, 4)]  # (gate_up, down) bits, layer by layer
MODEL_LAYERS = 48  # expert layers of the model the shape is taken from


def hbm_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return 6650.0, "fallback"


def measure(tokens_list, *, layers: int = 6, steps: int = 20, rank: int = 0, world: int = 1, device=None,
            dist=None, mode: str = "peer") -> list[dict]:
    """One result per token count.  ``dist`` given: expert-parallel over its ranks (every rank
    must call this with the same arguments); otherwise the whole layer on ``device``."""
    dev = torch.device(device if device is not None else "cuda")
    ep = dist is not None and world > 1
    peak, kind = hbm_peak_gbs()
    banks = [qwen3_moe_layer("cpu" if ep else dev, seed=3030 + i, bits_gate_up=WIDTHS[i % 6][0],
                             bits_down=WIDTHS[i % 6][1]) for i in range(layers)]
    if ep:
        from dynquant_b200.sharded import ExpertParallelMoE, expert_shard

        peer = None
        if mode == "peer":
            from dynquant_b200.peer import PeerExchange

            peer = PeerExchange(max(tokens_list) * 2048 * 4, device=dev)  # the largest piece: fp32 partial rows
        eps = [ExpertParallelMoE(expert_shard(l.gate_up, 2 * l.inter, l.num_experts, rank, world).to(dev),
                                 expert_shard(l.down, l.hidden, l.num_experts, rank, world).to(dev),
                                 num_experts=l.num_experts, peer=peer) for l in banks]
    results = []
    for tokens in tokens_list:
        if ep and (tokens % world or tokens // world == 0):
            continue
        t_local = tokens // world if ep else tokens
        ids_all, w_all = seeded_routing(tokens, 128, 8, seed=99 + tokens)
        mine = slice(rank * t_local, (rank + 1) * t_local) if ep else slice(0, tokens)
        ids, w = ids_all[mine].to(dev).contiguous(), w_all[mine].to(dev).contiguous()
        x = torch.randn(t_local, 2048, device=dev).to(torch.bfloat16)
        scratch = torch.empty(ops.moe_scratch_bytes(max(tokens, 1), 8, 2048, 768, 128, torch.bfloat16),
                              dtype=torch.uint8, device=dev)

        def step():
            for i in range(layers):
                if ep:
                    eps[i](x, ids, w, mode=mode)
                else:
                    ops.moe_gemv(x, ids, w, banks[i].gate_up, banks[i].down, num_experts=128, scratch=scratch)

        before = ops.launch_count()
        for _ in range(3):
            step()
        launches_per_layer = (ops.launch_count() - before) / 3 / layers
        torch.cuda.synchronize(dev)
        # A CUDA graph of the step is replayed, so that the time is the device's -- on one GPU and,
        # with the exchanges over peer memory (kernel launches), expert-parallel too.  With the NCCL
        # exchanges the step runs eagerly: they are issued from Python rank by rank and the time
        # includes that host work.
        run, launch = step, "eager"
        if not ep or mode == "peer":  # (peer exchanges are kernel launches: the layer captures whole)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            graph.replay()
            torch.cuda.synchronize(dev)
            run, launch = graph.replay, "cuda graph"
        if ep:
            dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            run()
        stop.record()
        torch.cuda.synchronize(dev)
        seconds = start.elapsed_time(stop) / 1e3 / steps / layers
        if ep:
            t = torch.tensor([seconds], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            seconds = float(t.item())
        if ep and mode == "peer":
            peer.check()  # no exchange's bounded wait ran out
        nbytes = sum(l.bytes_for(ids_all, tokens) for l in banks) / layers
        results.append({
            "workload": "qwen3-30b-a3b expert layer (128 experts, top-8, hidden 2048, inter 768, 2/3/4-bit banks)",
            "tokens": tokens, "n_gpus": world,
            "exchange": mode if ep else None, "launch": launch, "layers_timed": layers,
            "launches_per_layer": round(launches_per_layer, 2),
            "us_per_layer": round(seconds * 1e6, 2), "tokens_per_s_per_layer": round(tokens / seconds, 1),
            "tokens_per_s": round(tokens / seconds / MODEL_LAYERS, 1),
            "activated_experts": int(torch.unique(ids_all).numel()),
            "algorithmic_mb_per_layer": round(nbytes / 1e6, 2), "gbps": round(nbytes / seconds / 1e9, 1),
            "frac_of_hbm_peak": round(nbytes / seconds / 1e9 / (peak * world), 4),
            "peak": f"{peak} GB/s per GPU ({kind})",
        })
    return results


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,2,4,8,16,32,64")
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--ep", action="store_true", help="expert-parallel over the torchrun ranks")
    ap.add_argument("--mode", default="peer", choices=["peer", "all_to_all", "replicated"])
    ns = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if ns.ep:
        import datetime

        import torch.distributed as dist_mod

        dist = dist_mod
        # a short timeout: a rank that fails must end the others' next collective, not hang them
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    out = measure([int(t) for t in ns.tokens.split(",")], layers=ns.layers, steps=ns.steps, rank=rank,
                  world=world if ns.ep else 1, device=dev, dist=dist, mode=ns.mode)
    if rank == 0:
        for row in out:
            print(json.dumps(row), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
