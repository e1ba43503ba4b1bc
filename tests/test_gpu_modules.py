"""Packed modules and serving-plugin methods on the GPU, against dense reconstructions.

Follows the reference's module tests (tests/test_runtime_linear.py:58-120, :136-185): a packed
module equals ``F.linear`` on the dequantized weight, leading dims are kept, tied tables share
one buffer, state_dict keys are ``qweight/scales/offsets/bias``."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import TAG, make_quant, raw

pytestmark = pytest.mark.gpu


def dense_ref(x, qt, bias=None):
    from oracle import oracle as O

    y = O.c_gemv(raw(x.reshape(-1, qt.in_features)), TAG[x.dtype], raw(qt.packed), raw(qt.scales), raw(qt.offsets),
                 TAG[qt.scales.dtype], O.geometry(qt.bits, qt.group_size, qt.in_features))
    y = torch.from_numpy(y)
    if bias is not None:
        y = y + bias.float().cpu()
    return y.reshape(*x.shape[:-1], qt.num_rows)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_linear_module_equals_dense_reconstruction(bits):
    from dynquant_b200.runtime import DynQuantLinear

    qt = make_quant(96, 512, 128, bits, torch.float16).to("cuda")
    bias = torch.randn(96, dtype=torch.float16, device="cuda")
    mod = DynQuantLinear(qt, bias)
    assert set(mod.state_dict()) == {"qweight", "scales", "offsets", "bias"}
    # decode, leading dims, several GEMV launches (9..64 rows), dequantize + dense (> 64 rows)
    for shape in ((1, 512), (2, 3, 512), (20, 512), (70, 512)):
        x = torch.randn(*shape, dtype=torch.float16, device="cuda")
        got = mod(x)
        assert got.shape == (*shape[:-1], 96) and got.dtype == torch.float16
        want = dense_ref(x, qt, bias)
        torch.testing.assert_close(got.float().cpu(), want, rtol=2e-2, atol=5e-3 * float(want.abs().max()))


def test_embedding_lookup_and_tied_table():
    from dynquant_b200.runtime import DynQuantEmbedding, DynQuantLinear, packed_bytes

    qt = make_quant(300, 256, -1, 4, torch.float16).to("cuda")  # per-row table
    emb = DynQuantEmbedding(qt)
    head = DynQuantLinear(qt, tied_to=emb)
    assert head.holder is emb and head.weight_qt.packed.data_ptr() == emb.weight_qt.packed.data_ptr()
    ids = torch.tensor([[0, 7, 299], [5, 5, 1]], device="cuda")
    rows = emb(ids)
    dense = qt.dequantize()
    assert rows.shape == (2, 3, 256)
    assert torch.equal(rows, dense[ids.reshape(-1)].reshape(2, 3, 256))
    x = torch.randn(1, 256, dtype=torch.float16, device="cuda")
    torch.testing.assert_close(head(x).float().cpu(), dense_ref(x, qt), rtol=2e-2, atol=2e-2)
    holder = torch.nn.ModuleList([emb, head])
    assert packed_bytes(holder) == qt.nbytes  # tied table counted once


def test_fused_layer_with_mixed_widths_and_bias_in_one_call():
    from dynquant_b200.plugin import DynQuantLinearMethod, ShardSpec

    specs = [ShardSpec("q_proj", 4, 128, 256), ShardSpec("k_proj", 2, 128, 64), ShardSpec("v_proj", 3, 128, 64)]
    method = DynQuantLinearMethod(None, specs)
    layer = torch.nn.Module()
    method.create_weights(layer, 512, [256, 64, 64], 512, 384, torch.float16, device="cuda")
    parts = [make_quant(s.out_features, 512, 128, s.bits, torch.float16, seed=10 + i).to("cuda")
             for i, s in enumerate(specs)]
    for i, qt in enumerate(parts):
        method.load_shard(layer, i, qt)
    bias = torch.randn(384, dtype=torch.bfloat16, device="cuda")
    for m in (1, 3, 8, 12, 66):
        x = torch.randn(m, 512, dtype=torch.bfloat16, device="cuda")
        got = method.apply(layer, x, bias)
        want = torch.cat([dense_ref(x, qt) for qt in parts], dim=-1) + bias.float().cpu()
        assert got.shape == (m, 384) and got.dtype == torch.bfloat16
        # bf16 output: half an ulp of the largest value; the > 64-row path also rounds the
        # dequantized weight to bf16 before the dense matmul, like the reference's torch path
        atol = (2e-2 if m > 64 else 5e-3) * float(want.abs().max())
        torch.testing.assert_close(got.float().cpu(), want, rtol=2e-2, atol=atol)


def test_moe_method_matches_the_oracle():
    from dynquant_b200.plugin import DynQuantMoEMethod
    from dynquant_b200.workloads import qwen3_moe_layer, seeded_routing
    from oracle import oracle as O

    experts, hidden, inter, topk = 8, 512, 256, 2
    bank = qwen3_moe_layer("cuda", seed=9, bits_gate_up=3, bits_down=4, num_experts=experts, hidden=hidden,
                           inter=inter, topk=topk)
    method = DynQuantMoEMethod(None, bits_gate_up=3, bits_down=4)
    layer = torch.nn.Module()
    method.create_weights(layer, experts, hidden, inter, torch.float16, device="cuda")
    method.load_banks(layer, bank.gate_up, bank.down)
    ids, w = seeded_routing(6, experts, topk, seed=2)
    x = torch.randn(6, hidden, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    got = method.apply(layer, x.cuda(), w.cuda(), ids.cuda())

    def b(qt):
        return (raw(qt.packed), raw(qt.scales), raw(qt.offsets), "f16", O.geometry(qt.bits, 128, qt.in_features))

    want = O.c_moe(raw(x), "bf16", ids.numpy(), w.numpy(), b(bank.gate_up), b(bank.down), inter=inter,
                   num_experts=experts, h_round="bf16")
    err = np.linalg.norm(got.float().cpu().numpy() - want) / np.linalg.norm(want)
    assert err <= 5e-3  # bf16 output rounding on top of the 2e-3 of the fp32 path


def test_gemv_sequence_and_step_runner_match_individual_calls():
    from dynquant_b200 import ops
    from dynquant_b200.stack import StepRunner
    from dynquant_b200.workloads import qwen2b_stack

    stack = qwen2b_stack(device="cuda", layers=1, vocab=4096)
    runner = StepRunner(stack, 2, device="cuda")
    runner.run()
    torch.cuda.synchronize()
    eager = {k: v.clone() for k, v in runner.outputs.items()}
    # a fused launch may slice the reduction axis differently from the single call: the two
    # agree to the rounding of the fp32 partial sums, i.e. within one bf16 ulp of the output
    for mod in stack.modules:
        want = ops.quantized_matmul(runner.inputs[mod.input], mod.weight)
        diff = (eager[mod.name].float() - want.float()).abs()
        bound = want.float().abs() * 2.0**-7 + 1e-4 * want.float().abs().max()
        assert bool((diff <= bound).all()), (mod.name, float(diff.max()))
    for mode in ("dataflow", "chain", "independent"):
        for v in runner.outputs.values():
            v.zero_()
        runner.capture(mode)
        runner.replay()
        torch.cuda.synchronize()
        for name, want in eager.items():
            if mode == "independent":  # single launches: may slice the reduction differently
                diff = (runner.outputs[name].float() - want.float()).abs()
                assert bool((diff <= want.float().abs() * 2.0**-7 + 1e-4 * want.float().abs().max()).all()), name
            else:
                assert torch.equal(runner.outputs[name], want), (mode, name)


@pytest.mark.parametrize("rows_m", [1, 8])
def test_a_step_with_cluster_launches_in_its_graph_matches_the_eager_step(rows_m):
    """One layer of the 14B set: its down-projection (5120 x 17408) takes the streaming body sliced
    over a thread-block cluster.  Cluster launches with programmatic dependent launch between
    them, captured into a graph: the same bits as the eager step, every module within the
    rounding of a re-sliced sum of the single call."""
    from dynquant_b200 import ops
    from dynquant_b200.stack import StepRunner
    from dynquant_b200.workloads import qwen14b_linear_set

    stack = qwen14b_linear_set(device="cuda", layers=1)
    runner = StepRunner(stack, rows_m, device="cuda")
    runner.run()
    torch.cuda.synchronize()
    eager = {k: v.clone() for k, v in runner.outputs.items()}
    kernels = set()
    for mod in stack.modules:
        want = ops.quantized_matmul(runner.inputs[mod.input], mod.weight)
        kernels.add(ops.last_kernel())
        diff = (eager[mod.name].float() - want.float()).abs()
        bound = want.float().abs() * 2.0**-7 + 1e-4 * want.float().abs().max()
        assert bool((diff <= bound).all()), (mod.name, float(diff.max()))
    assert "gemv_mma_stream_sliced_kernel" in kernels, kernels
    for mode in ("dataflow", "chain"):
        for v in runner.outputs.values():
            v.zero_()
        runner.capture(mode)
        runner.replay()
        runner.replay()
        torch.cuda.synchronize()
        for name, want in eager.items():
            assert torch.equal(runner.outputs[name], want), (mode, name)


def test_gemv_host_entry_point_round_trips_through_pinned_memory():
    from dynquant_b200 import ops

    qt = make_quant(128, 512, 128, 4, torch.float16).to("cuda")
    x_host = torch.randn(2, 512).to(torch.bfloat16).pin_memory()
    out_host = torch.empty(2, 128, dtype=torch.bfloat16).pin_memory()
    x_dev = torch.empty(2, 512, dtype=torch.bfloat16, device="cuda")
    out_dev = torch.empty(2, 128, dtype=torch.bfloat16, device="cuda")
    ops.gemv_host(x_host, qt, out_host, x_dev, out_dev)
    want = ops.gemv(x_host.cuda(), qt.packed, qt.scales, qt.offsets, 4, 128, 512)
    assert torch.equal(out_host, want.cpu())


def test_step_graph_with_its_copies_matches_the_plain_step():
    """``capture_with_io``: host -> device copies, the step and the read-back in one graph give
    what the same step gives on resident inputs."""
    from dynquant_b200.stack import StepRunner
    from dynquant_b200.workloads import qwen2b_stack

    stack = qwen2b_stack(device="cuda", layers=1, vocab=1024)
    runner = StepRunner(stack, 2, device="cuda")
    runner.run()
    torch.cuda.synchronize()
    last = stack.modules[-1].name
    expect = runner.outputs[last].clone()
    host_in = {k: v.cpu().pin_memory() for k, v in runner.inputs.items()}
    host_out = torch.zeros_like(expect, device="cpu").pin_memory()
    for v in runner.inputs.values():
        v.zero_()  # the graph must bring the activations back from the host
    runner.capture_with_io(host_in, last, host_out)
    for v in runner.inputs.values():
        v.zero_()
    runner.outputs[last].zero_()
    runner.replay_with_io()
    torch.cuda.synchronize()
    assert torch.equal(host_out, expect.cpu())
    with pytest.raises(ValueError, match="pinned"):
        runner.capture_with_io({k: v.cpu() for k, v in runner.inputs.items()}, last, host_out)


def test_vllm_adapter_layer_loads_through_the_placement_hooks_and_runs_one_launch():
    """The adapter vLLM builds layers from: parameters created by ``create_weights`` on the GPU,
    filled through vLLM's v2 loader hooks (a fused q/k/v layer of three widths), applied with a
    bias -- one kernel launch -- and compared with the oracle."""
    pytest.importorskip("vllm", reason="the adapter needs vLLM")
    from conftest import vllm_world_of_one

    from dynquant_b200 import ops
    from dynquant_b200.checkpoint import ModuleSpec
    from dynquant_b200.vllm_plugin import DynQuantLinearMethod

    vllm_world_of_one()
    k = 1024
    widths = [("q_proj", 4, 512), ("k_proj", 2, 128), ("v_proj", 3, 128)]
    parts = [make_quant(rows, k, 128, bits, torch.float16, seed=20 + bits) for _, bits, rows in widths]
    layer = torch.nn.Module()
    method = DynQuantLinearMethod(None, [(f"l.{n}", ModuleSpec(bits=b)) for n, b, _ in widths])
    with torch.device("cuda"):
        method.create_weights(layer, input_size_per_partition=k, output_partition_sizes=[r for *_, r in widths],
                              input_size=k, output_size=768, params_dtype=torch.float16, weight_loader=None)
    assert layer.qweight.is_cuda
    offset = 0
    for (name, _, rows), qt in zip(widths, parts):
        for attr, source in (("qweight", qt.packed), ("scales", qt.scales), ("offsets", qt.offsets)):
            getattr(layer, attr).load_qkv_weight(loaded_weight=source.cuda(), shard_offset=offset, shard_size=rows,
                                                 shard_id=name[0], num_heads=1)
        offset += rows
    bias = torch.randn(768, dtype=torch.bfloat16, device="cuda")
    x = torch.randn(3, k, dtype=torch.bfloat16, device="cuda")
    before = ops.launch_count()
    got = method.apply(layer, x, bias)
    assert ops.launch_count() - before == 1
    want = torch.cat([dense_ref(x, qt) for qt in parts], dim=-1) + bias.float().cpu()
    torch.testing.assert_close(got.float().cpu(), want, rtol=2e-2, atol=5e-3 * float(want.abs().max()))
