"""The multi-GPU placement logic on CPU: two gloo ranks as child processes, the CPU oracle
standing in for the kernels.  Checks that column shards and expert shards reassemble to the
single-device result for both MoE exchange modes."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def _raw(t):
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.int32:
        return t.numpy().view(np.uint32)
    return t.numpy()


TAG = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}


def _oracle_matmul(x, qt):
    from oracle import oracle as O

    y = O.c_gemv(_raw(x), TAG[x.dtype], _raw(qt.packed), _raw(qt.scales), _raw(qt.offsets), TAG[qt.scales.dtype],
                 O.geometry(qt.bits, qt.group_size, qt.in_features))
    return torch.from_numpy(y)


def _oracle_moe(hidden, inter):
    def compute(x, ids, w, gate_up, down, num_experts):
        from oracle import oracle as O

        def bank(qt):
            return (_raw(qt.packed), _raw(qt.scales), _raw(qt.offsets), TAG[qt.scales.dtype],
                    O.geometry(qt.bits, qt.group_size, qt.in_features))

        y = O.c_moe(_raw(x), TAG[x.dtype], ids.numpy(), w.numpy(), bank(gate_up), bank(down), inter=inter,
                    num_experts=num_experts, h_round=TAG[x.dtype])
        return torch.from_numpy(y)

    return compute


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from dynquant_b200.format import QuantTensor
        from dynquant_b200.sharded import (ColumnShardedLinear, ExpertParallelMoE, InputShardedLinear, column_shard,
                                           expert_shard, input_shard)
        from dynquant_b200.workloads import random_quant_tensor, seeded_routing

        gen = torch.Generator().manual_seed(5)
        # ---- column-sharded dense ----
        qt = random_quant_tensor(64, 256, 3, generator=gen)
        x = torch.randn(2, 256, generator=gen).to(torch.bfloat16)
        full = _oracle_matmul(x, qt)
        layer = ColumnShardedLinear(column_shard(qt, rank, world), compute=_oracle_matmul)
        got = layer(x)
        ok_dense = bool(torch.equal(got, full))
        # ---- input-sharded dense (K split on group boundaries, partial sums all-reduced) ----
        errs_in = {}
        for bits in (2, 3, 4, 8):
            wide = random_quant_tensor(48, 512, bits, generator=gen)
            xw = torch.randn(3, 512, generator=gen).to(torch.bfloat16)
            bias = torch.randn(48, generator=gen)
            want_in = _oracle_matmul(xw, wide) + bias
            part = input_shard(wide, rank, world)
            k_local = 512 // world
            layer_in = InputShardedLinear(part, bias=bias, compute=_oracle_matmul)
            y_in = layer_in(xw[:, rank * k_local : (rank + 1) * k_local].contiguous()).float()
            ref_in = want_in.to(torch.bfloat16).float()
            errs_in[bits] = float((y_in - ref_in).abs().max() / ref_in.abs().max())
            assert part.in_features == k_local and part.packed.shape == (48, k_local * bits // 32)
        # ---- expert parallel ----
        experts, hidden, inter, topk, t_local = 4, 256, 128, 2, 3
        gate_up = random_quant_tensor(experts * 2 * inter, hidden, 4, generator=gen)
        down = random_quant_tensor(experts * hidden, inter, 3, generator=gen)
        ids_all, w_all = seeded_routing(world * t_local, experts, topk, seed=8)
        x_all = torch.randn(world * t_local, hidden, generator=gen).to(torch.bfloat16)
        want = _oracle_moe(hidden, inter)(x_all, ids_all, w_all, gate_up, down, experts)
        mine = slice(rank * t_local, (rank + 1) * t_local)
        ep = ExpertParallelMoE(expert_shard(gate_up, 2 * inter, experts, rank, world),
                               expert_shard(down, hidden, experts, rank, world), num_experts=experts,
                               compute=_oracle_moe(hidden, inter))
        errs = {}
        for mode in ("all_to_all", "replicated"):
            y = ep(x_all[mine], ids_all[mine], w_all[mine], mode=mode).float()
            ref = want[mine].to(torch.bfloat16).float()
            errs[mode] = float((y - ref).abs().max() / (ref.abs().max() + 1e-30))
        # ---- more gathered tokens than one call of the grouped kernel takes: chunks of 64 ----
        t_big = 40  # 80 gathered tokens over two ranks
        ids_big, w_big = seeded_routing(world * t_big, experts, topk, seed=9)
        x_big = torch.randn(world * t_big, hidden, generator=gen).to(torch.bfloat16)
        want_big = _oracle_moe(hidden, inter)(x_big, ids_big, w_big, gate_up, down, experts)
        inner = _oracle_moe(hidden, inter)

        def bounded(x, ids, w, gu, dn, n):
            assert x.shape[0] <= 64, f"{x.shape[0]} tokens in one call"
            return inner(x, ids, w, gu, dn, n)

        ep_big = ExpertParallelMoE(expert_shard(gate_up, 2 * inter, experts, rank, world),
                                   expert_shard(down, hidden, experts, rank, world), num_experts=experts,
                                   compute=bounded, max_tokens=64)
        big = slice(rank * t_big, (rank + 1) * t_big)
        for mode in ("all_to_all", "replicated"):
            y = ep_big(x_big[big], ids_big[big], w_big[big], mode=mode).float()
            ref = want_big[big].to(torch.bfloat16).float()
            errs[mode + "/80 tokens"] = float((y - ref).abs().max() / (ref.abs().max() + 1e-30))
        results[rank] = (ok_dense, errs, errs_in)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_reassembles_to_the_single_device_result():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        ok_dense, errs, errs_in = results[rank]
        assert ok_dense, f"rank {rank}: gathered column shards differ from the unsharded result"
        for bits, err in errs_in.items():
            assert err <= 1e-2, f"rank {rank} input-sharded {bits}-bit: {err}"  # one bf16 rounding of the output
        for mode, err in errs.items():
            assert err <= 1e-2, f"rank {rank} {mode}: {err}"  # one bf16 rounding of the output


def test_shard_helpers_reject_uneven_splits():
    from dynquant_b200.sharded import column_shard, expert_shard
    from dynquant_b200.workloads import random_quant_tensor

    qt = random_quant_tensor(10, 128, 4)
    with pytest.raises(ValueError):
        column_shard(qt, 0, 4)
    with pytest.raises(ValueError):
        expert_shard(qt, 2, 5, 0, 2)
    part = column_shard(qt, 1, 2)
    assert part.num_rows == 5 and part.row_offset == 5
    from dynquant_b200.sharded import input_shard

    with pytest.raises(ValueError, match="group boundaries"):
        input_shard(random_quant_tensor(4, 384, 4), 0, 2)  # three groups over two ranks
    with pytest.raises(ValueError, match="per-row"):
        input_shard(random_quant_tensor(4, 256, 4, group_size=-1), 0, 2)
