"""MoE grouped GEMV against the composition oracle (the reference has no MoE kernel; the
oracle is its per-expert dequantize + matmul definition, ``oracle/dq_oracle.c::dqo_moe``)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import TAG, raw
from test_gpu_parity import within_one_ulp_16

pytestmark = pytest.mark.gpu


def bank_for_oracle(qt):
    from oracle import oracle as O

    return (raw(qt.packed), raw(qt.scales), raw(qt.offsets), TAG[qt.scales.dtype],
            O.geometry(qt.bits, qt.group_size, qt.in_features))


def run_case(tokens, experts, hidden, inter, topk, bits_gu, bits_dn, act=torch.bfloat16, seed=1, local=None):
    from dynquant_b200 import ops
    from dynquant_b200.workloads import qwen3_moe_layer, seeded_routing
    from oracle import oracle as O

    layer = qwen3_moe_layer("cuda", seed=seed, bits_gate_up=bits_gu, bits_down=bits_dn, num_experts=experts,
                            hidden=hidden, inter=inter, topk=topk)
    ids, w = seeded_routing(tokens, experts, topk, seed=seed + 7)
    if local is not None:  # an expert-parallel rank: experts outside [lo, hi) are not held here
        lo, hi = local
        ids = torch.where((ids >= lo) & (ids < hi), ids, torch.full_like(ids, -1))
    x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(seed)).to(act)
    got = ops.moe_gemv(x.cuda(), ids.cuda(), w.cuda(), layer.gate_up, layer.down, num_experts=experts,
                       out_dtype=torch.float32)
    want = O.c_moe(raw(x), TAG[act], ids.numpy(), w.numpy(), bank_for_oracle(layer.gate_up),
                   bank_for_oracle(layer.down), inter=inter, num_experts=experts, h_round=TAG[act])
    return got.cpu().numpy(), want, layer, ids, w, x


@pytest.mark.parametrize("tokens", [1, 2, 3, 4, 5, 8, 16, 32, 33, 64])
@pytest.mark.parametrize(("bits_gu", "bits_dn"), [(2, 4), (3, 3), (4, 2), (8, 8)])
def test_moe_matches_the_composition_oracle(tokens, bits_gu, bits_dn):
    got, want, *_ = run_case(tokens, 16, 512, 256, 4, bits_gu, bits_dn)
    scale = np.abs(want).max() + 1e-30
    # the intermediate is rounded to bf16 on both sides; one-ulp flips of it are the noise floor
    assert np.abs(got - want).max() / scale <= 4e-3
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-3


def test_moe_qwen3_shape_fp16_and_determinism():
    from dynquant_b200 import ops

    got, want, layer, ids, w, x = run_case(4, 128, 2048, 768, 8, 3, 4, act=torch.float16, seed=3)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-3
    first = ops.moe_gemv(x.cuda(), ids.cuda(), w.cuda(), layer.gate_up, layer.down, num_experts=128)
    for _ in range(4):
        again = ops.moe_gemv(x.cuda(), ids.cuda(), w.cuda(), layer.gate_up, layer.down, num_experts=128)
        assert torch.equal(first, again)
    assert first.dtype == torch.float16


def test_moe_qwen3_shape_at_thirty_two_tokens():
    """The real expert shape where the launcher switches to its 80-register build (three CTAs
    per SM), whole rows per warp and eight staged rows."""
    got, want, *_ = run_case(32, 128, 2048, 768, 8, 2, 4, seed=11)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-3


def test_moe_skips_experts_that_are_not_local():
    got, want, *_ = run_case(8, 16, 512, 256, 4, 4, 4, local=(4, 8))
    assert np.linalg.norm(got - want) / (np.linalg.norm(want) + 1e-30) <= 2e-3


def test_moe_with_no_local_expert_at_all_writes_zeros():
    """Every id outside [0, num_experts) -- an expert-parallel rank that owns none of the experts
    a batch was routed to: the output is zero (and is written: it starts as garbage here)."""
    from dynquant_b200 import ops
    from dynquant_b200.workloads import qwen3_moe_layer

    layer = qwen3_moe_layer("cuda", seed=5, num_experts=4, hidden=256, inter=128, topk=2)
    ids = torch.full((3, 2), -1, dtype=torch.int32, device="cuda")
    w = torch.full((3, 2), 0.5, device="cuda")
    x = torch.randn(3, 256, device="cuda").to(torch.bfloat16)
    scratch = torch.full((ops.moe_scratch_bytes(3, 2, 256, 128, 4, torch.bfloat16),), 0xAB, dtype=torch.uint8, device="cuda")
    for _ in range(2):  # the second call reuses the scratch the first one left behind
        got = ops.moe_gemv(x, ids, w, layer.gate_up, layer.down, num_experts=4, scratch=scratch)
        assert got.shape == (3, 256) and not bool(got.float().abs().max() > 0)


def test_moe_reuses_scratch_that_starts_as_garbage():
    """The per-group counters of the fused combine live in caller scratch: never-initialised
    memory, and memory left behind by a previous call of another size, must both work."""
    from dynquant_b200 import ops
    from dynquant_b200.workloads import qwen3_moe_layer, seeded_routing

    layer = qwen3_moe_layer("cuda", seed=6, bits_gate_up=3, bits_down=4, num_experts=8, hidden=512, inter=256, topk=2)
    scratch = torch.full((ops.moe_scratch_bytes(16, 2, 512, 256, 8, torch.bfloat16),), 0xCD, dtype=torch.uint8, device="cuda")
    for tokens in (16, 3, 9):
        ids, w = seeded_routing(tokens, 8, 2, seed=tokens)
        x = torch.randn(tokens, 512, generator=torch.Generator().manual_seed(tokens)).to(torch.bfloat16).cuda()
        with_scratch = ops.moe_gemv(x, ids.cuda(), w.cuda(), layer.gate_up, layer.down, num_experts=8, scratch=scratch)
        fresh = ops.moe_gemv(x, ids.cuda(), w.cuda(), layer.gate_up, layer.down, num_experts=8)
        assert torch.equal(with_scratch, fresh)


def test_moe_many_tokens_on_one_expert():
    """More than eight tokens on one expert: the expert's rows are streamed once per 8 tokens."""
    from dynquant_b200 import ops
    from dynquant_b200.workloads import qwen3_moe_layer
    from oracle import oracle as O

    layer = qwen3_moe_layer("cuda", seed=5, bits_gate_up=4, bits_down=3, num_experts=4, hidden=256, inter=128, topk=2)
    tokens = 21
    ids = torch.tensor([[0, 1 + (t % 3)] for t in range(tokens)], dtype=torch.int32)
    w = torch.full((tokens, 2), 0.5)
    x = torch.randn(tokens, 256, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    got = ops.moe_gemv(x.cuda(), ids.cuda(), w.cuda(), layer.gate_up, layer.down, num_experts=4,
                       out_dtype=torch.float32).cpu().numpy()
    want = O.c_moe(raw(x), "bf16", ids.numpy(), w.numpy(), bank_for_oracle(layer.gate_up),
                   bank_for_oracle(layer.down), inter=128, num_experts=4, h_round="bf16")
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-3


def test_moe_rejects_bad_arguments():
    from dynquant_b200 import ops
    from dynquant_b200.workloads import qwen3_moe_layer, seeded_routing

    layer = qwen3_moe_layer("cuda", num_experts=4, hidden=256, inter=128, topk=2)
    ids, w = seeded_routing(65, 4, 2)
    x = torch.randn(65, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="exceeds the limit"):
        ops.moe_gemv(x, ids.cuda(), w.cuda(), layer.gate_up, layer.down, num_experts=4)
    ids, w = seeded_routing(2, 4, 2)
    with pytest.raises(RuntimeError, match="folded to rows"):
        ops.moe_gemv(x[:2].contiguous(), ids.cuda(), w.cuda(), layer.down, layer.gate_up, num_experts=4)


def test_moe_qwen3_shape_at_sixty_four_tokens():
    """BASELINE's MoE configuration at its largest step: 128 experts, top-8, hidden 2048,
    intermediate 768, 64 tokens (512 assignments, nearly every expert active)."""
    got, want, *_ = run_case(64, 128, 2048, 768, 8, 3, 2, seed=21)
    scale = np.abs(want).max() + 1e-30
    assert np.abs(got - want).max() / scale <= 4e-3
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-3


@pytest.mark.parametrize("act", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize(("bits_gu", "bits_dn"), [(2, 4), (3, 3), (4, 2), (8, 8)])
def test_moe_stage_by_stage(act, bits_gu, bits_dn):
    """Where the end-to-end distance comes from.  The call's scratch holds both intermediates:
    ``h = silu(g) * u`` per assignment, rounded once to the activation dtype, and the fp32 down
    projection ``d`` per assignment.  Checked separately:

    * h is the oracle's fp32 ``silu(g) * u`` rounded once, give or take one unit in the last
      place (with fp16 activations that is inside 1e-3 normwise; bf16's unit is 2^-8);
    * d, computed by the oracle FROM THE KERNEL'S OWN h, is within 1e-3: the down stage adds
      nothing beyond accumulation noise;
    * y is the weighted sum of the kernel's own d rows, in slot order, to fp32 rounding.

    So all of the layer's distance from an unrounded oracle is the one rounding of h."""
    from dynquant_b200 import ops
    from dynquant_b200.workloads import qwen3_moe_layer, seeded_routing
    from oracle import oracle as O

    tokens, experts, hidden, inter, topk = 12, 16, 512, 256, 4
    layer = qwen3_moe_layer("cuda", seed=31, bits_gate_up=bits_gu, bits_down=bits_dn, num_experts=experts,
                            hidden=hidden, inter=inter, topk=topk)
    ids, w = seeded_routing(tokens, experts, topk, seed=5)
    x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(4)).to(act)
    need = ops.moe_scratch_bytes(tokens, topk, hidden, inter, experts, act)
    scratch = torch.zeros(need, dtype=torch.uint8, device="cuda")
    y = ops.moe_gemv(x.cuda(), ids.cuda(), w.cuda(), layer.gate_up, layer.down, num_experts=experts,
                     out_dtype=torch.float32, scratch=scratch)
    torch.cuda.synchronize()
    n_assign = tokens * topk
    h_bytes = n_assign * inter * 2
    h = scratch[:h_bytes].view(act).view(n_assign, inter).cpu()
    d_off = (h_bytes + 255) // 256 * 256
    d = scratch[d_off:d_off + n_assign * hidden * 4].view(torch.float32).view(n_assign, hidden).cpu()

    def expert_rows(bank, e, rows_per_expert):
        part = bank.rows(e * rows_per_expert, (e + 1) * rows_per_expert)
        return (raw(part.packed), raw(part.scales), raw(part.offsets), TAG[part.scales.dtype],
                O.geometry(part.bits, part.group_size, part.in_features))

    h_err2 = h_ref2 = 0.0
    for t in range(tokens):
        for k in range(topk):
            e, aid = int(ids[t, k]), t * topk + k
            packed, scales, offsets, tag, geom = expert_rows(layer.gate_up, e, 2 * inter)
            gu = O.c_gemv(raw(x[t:t + 1]), TAG[act], packed, scales, offsets, tag, geom)[0]
            g, u = gu[:inter].astype(np.float64), gu[inter:].astype(np.float64)
            h32 = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
            got_h = h[aid].float().numpy()
            # the oracle's value rounded once, give or take one unit in the last place; plus the
            # suite's usual absolute room for outputs that nearly cancel (2e-5 of the largest)
            assert within_one_ulp_16(h[aid:aid + 1], h32[None, :]), (t, k)
            h_err2 += float(((got_h - h32) ** 2).sum())
            h_ref2 += float((h32 ** 2).sum())
            packed, scales, offsets, tag, geom = expert_rows(layer.down, e, hidden)
            want_d = O.c_gemv(raw(h[aid:aid + 1]), TAG[act], packed, scales, offsets, tag, geom)[0]
            got_d = d[aid].numpy()
            assert np.abs(got_d - want_d).max() / (np.abs(want_d).max() + 1e-30) <= 1e-3, (t, k)
            assert np.linalg.norm(got_d - want_d) / (np.linalg.norm(want_d) + 1e-30) <= 1e-3, (t, k)
    if act == torch.float16:
        assert (h_err2 / h_ref2) ** 0.5 <= 1e-3  # fp16's rounding itself is inside the bar
    combined = (w.double().reshape(n_assign, 1) * d.double()).reshape(tokens, topk, hidden).sum(1)
    assert float((y.cpu().double() - combined).abs().max()) <= 1e-5 * float(combined.abs().max())


@pytest.mark.parametrize(("tokens", "launches"), [(1, 2), (2, 2), (4, 2), (5, 3)])
def test_few_tokens_take_the_down_projection_with_the_combine_folded_in(tokens, launches):
    """Up to four tokens the layer is two launches: the down projection runs token by token (a
    warp per expert of the token) and its cross-warp sum is the combine.  Real expert shape."""
    from dynquant_b200 import _lib, ops

    before = int(_lib.load().dq_launch_count())
    got, want, *_ = run_case(tokens, 128, 2048, 768, 8, 3, 4, seed=40 + tokens)
    assert int(_lib.load().dq_launch_count()) - before == launches
    if launches == 2:
        assert ops.last_kernel() == "moe_down_token_kernel"
    scale = np.abs(want).max() + 1e-30
    assert np.abs(got - want).max() / scale <= 4e-3
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-3


@pytest.mark.parametrize("bits_dn", [2, 3, 4, 8])
def test_few_tokens_every_width_dtype_and_absent_experts(bits_dn):
    from dynquant_b200 import ops

    for act in (torch.bfloat16, torch.float16):
        got, want, *_ = run_case(3, 16, 512, 256, 4, 4, bits_dn, act=act, seed=50 + bits_dn, local=(4, 12))
        assert ops.last_kernel() == "moe_down_token_kernel"
        assert np.linalg.norm(got - want) / (np.linalg.norm(want) + 1e-30) <= 2e-3
    # a reduction axis of three steps (odd): not this kernel's; the three-launch path takes it
    got, want, *_ = run_case(2, 8, 256, 384, 2, 4, bits_dn, seed=60)
    assert ops.last_kernel() != "moe_down_token_kernel"
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-3


@pytest.mark.parametrize("tokens", [2, 12])
def test_a_shard_of_the_experts_takes_global_ids(tokens):
    """One rank of an expert-parallel layer: banks of experts [4, 12) only, global ids and
    ``first_expert=4`` -- bit-identical to renumbering the ids on the host first."""
    from dynquant_b200 import ops
    from dynquant_b200.workloads import qwen3_moe_layer, seeded_routing

    layer = qwen3_moe_layer("cuda", seed=9, bits_gate_up=3, bits_down=4, num_experts=16, hidden=512, inter=256, topk=4)
    gate_up = layer.gate_up.rows(4 * 512, 12 * 512)
    down = layer.down.rows(4 * 512, 12 * 512)
    ids, w = seeded_routing(tokens, 16, 4, seed=tokens)
    x = torch.randn(tokens, 512, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    local = torch.where((ids >= 4) & (ids < 12), ids - 4, torch.full_like(ids, -1)).to(torch.int32)
    want = ops.moe_gemv(x, local.cuda(), w.cuda(), gate_up, down, num_experts=8, out_dtype=torch.float32)
    got = ops.moe_gemv(x, ids.to(torch.int32).cuda(), w.cuda(), gate_up, down, num_experts=8, out_dtype=torch.float32,
                       first_expert=4)
    assert torch.equal(got, want) and bool(want.abs().max() > 0)
