"""The sharded paths on real GPUs: this library's kernels + NCCL together (needs two devices).

The gloo tests (``test_sharded_gloo.py``) cover the placement logic with the oracle as the
compute; here every rank runs the CUDA kernels on its shard and the exchange is NCCL over
NVLink, and the reassembled result is compared with the same computation on one GPU:

* column-sharded dense: the all-gathered output equals the unsharded kernel's, bit for bit
  (rows are independent: a shard's rows are computed exactly as in the whole matrix);
* expert-parallel MoE, both exchange modes: equal to the single-GPU layer up to the order of
  the fp32 sum over ranks.

No rank faults or hangs on purpose: process groups carry a short timeout, NVLS is off.
"""

from __future__ import annotations

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank: int, world: int, port: int, results) -> None:
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=60))
    try:
        from dynquant_b200 import ops
        from dynquant_b200.sharded import ColumnShardedLinear, ExpertParallelMoE, column_shard, expert_shard
        from dynquant_b200.workloads import qwen3_moe_layer, random_quant_tensor, seeded_routing

        out = {}
        # ---- column-sharded dense, every width, a long and a short matrix ----
        for bits, rows in ((2, 40960), (3, 2048), (4, 6144), (8, 40960)):
            gen = torch.Generator(device=dev).manual_seed(100 + bits)  # same seed: same tensor on every rank
            qt = random_quant_tensor(rows, 2048, bits, device=dev, generator=gen)
            x = torch.randn(1, 2048, device=dev, generator=gen).to(torch.bfloat16)
            full = ops.quantized_matmul(x, qt)
            got = ColumnShardedLinear(column_shard(qt, rank, world))(x)
            out[f"dense{bits}"] = bool(torch.equal(got, full))
        # ---- expert parallel ----
        layer = qwen3_moe_layer(dev, seed=77, bits_gate_up=3, bits_down=4, num_experts=16, hidden=1024, inter=512, topk=4)
        t_local = 6
        ids_all, w_all = seeded_routing(world * t_local, 16, 4, seed=5)
        x_all = torch.randn(world * t_local, 1024, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(dev)
        want = ops.moe_gemv(x_all, ids_all.to(dev), w_all.to(dev), layer.gate_up, layer.down, num_experts=16,
                            out_dtype=torch.float32)
        ep = ExpertParallelMoE(expert_shard(layer.gate_up, 2 * 512, 16, rank, world),
                               expert_shard(layer.down, 1024, 16, rank, world), num_experts=16)
        mine = slice(rank * t_local, (rank + 1) * t_local)
        from dynquant_b200.peer import PeerExchange

        ep.peer = PeerExchange(t_local * 1024 * 4, device=dev)
        for mode in ("all_to_all", "replicated", "peer"):
            y = ep(x_all[mine], ids_all[mine].to(dev), w_all[mine].to(dev), mode=mode).float()
            ref = want[mine].to(torch.bfloat16).float()
            out[mode] = float((y - ref).abs().max() / ref.abs().max())
        # ---- the library's own exchanges over peer memory against NCCL's ----
        from dynquant_b200.peer import PeerExchange

        ex = PeerExchange(1 << 20, device=dev)
        for n in (64, 4096, 124160):  # a few token rows ... half of the 248,320-row head at one row
            piece = torch.randn(n, device=dev).to(torch.bfloat16)
            mine_out = torch.empty(world * n, dtype=torch.bfloat16, device=dev)
            ex.all_gather(piece, mine_out)
            nccl_out = torch.empty_like(mine_out)
            dist.all_gather_into_tensor(nccl_out, piece)
            ex.check()
            out[f"gather{n}"] = bool(torch.equal(mine_out, nccl_out))
            partial = torch.randn(world * n, device=dev)
            got_rs = torch.empty(n, dtype=torch.float32, device=dev)
            ex.reduce_scatter(partial, got_rs)
            want_rs = torch.empty(n, dtype=torch.float32, device=dev)
            dist.reduce_scatter_tensor(want_rs, partial.clone())
            ex.check()
            out[f"scatter{n}"] = bool(torch.allclose(got_rs, want_rs, rtol=1e-6, atol=1e-6))
        # many exchanges back to back, captured in a CUDA graph and replayed
        piece = torch.full((2048,), float(rank + 1), device=dev)
        gathered = torch.zeros(world * 2048, device=dev)
        ex.all_gather(piece, gathered)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(10):
                ex.all_gather(piece, gathered)
        for _ in range(5):
            graph.replay()
        ex.check()
        want = torch.cat([torch.full((2048,), float(r + 1), device=dev) for r in range(world)])
        out["graph"] = bool(torch.equal(gathered, want))
        # ---- a whole sharded decode step: every stage's all-gather folded into its GEMV launch ----
        from dynquant_b200.sharded import ShardedStepRunner
        from dynquant_b200.stack import StepRunner
        from dynquant_b200.workloads import qwen2b_stack

        stack = qwen2b_stack(device=dev, vocab=40960, layers=2)
        single = StepRunner(stack, 2, device=dev)
        single.run()
        torch.cuda.synchronize()
        for exchange in ("fused", "peer"):
            runner = ShardedStepRunner(stack, 2, rank=rank, world=world, device=dev, shard_min_bytes=0,
                                       exchange=exchange)
            for name, t in single.inputs.items():
                runner.inputs[name].copy_(t)
            same, close = True, True
            for step in range(3):  # the window halves alternate from step to step
                runner.run()
                runner.check()
                for name in runner.sharded:
                    # the transfer is exact: what arrived is what every rank computed (NCCL as the witness)
                    piece = runner.runner.outputs[name].contiguous()
                    witness = torch.empty(world, *piece.shape, dtype=piece.dtype, device=dev)
                    dist.all_gather_into_tensor(witness, piece)
                    if not torch.equal(runner.full_output(name), witness):
                        same = False
                        bad = (runner.full_output(name) != witness).nonzero()
                        out[f"step/{exchange}: {name}, step {step}: {bad.shape[0]} of {witness.numel()} values differ from "
                            f"what the ranks computed, first at {bad[0].tolist()}, last at {bad[-1].tolist()}"] = False
                    # and the values are the single-GPU ones up to the summation order of a differently
                    # sliced reduction axis (a slab is a smaller matrix): one rounding of the bf16 output
                    got, ref = runner.gathered(name).float(), single.outputs[name].float()
                    close = close and bool(((got - ref).abs() <= 2.0 ** -7 * ref.abs() + 1e-6).all())
            out[f"step/{exchange}"] = same
            out[f"step/{exchange}/within one rounding of the single-GPU step"] = close
            out[f"step/{exchange}/all modules sharded"] = len(runner.sharded) == len(stack.modules)
            if exchange == "fused":
                out["step/fused/no stage fell back"] = runner.fused_stages == runner.gathers_per_step
                out["step/fused/one launch per stage"] = runner.launches_per_step == runner.gathers_per_step
            del runner
        results[rank] = out
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_paths_on_two_gpus_match_one_gpu():
    world = 2
    port = 29600 + (os.getpid() % 1000)
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        for key, value in results[rank].items():
            if isinstance(value, bool):
                assert value, f"rank {rank}: {key} differs from the reference result"
            else:
                assert value <= 1e-2, f"rank {rank} {key}: {value}"  # one bf16 rounding of the output
