"""The allocation-free MoE entry point (``dq_moe_gemv_static``), called through the C ABI.

Some hosts of this library cannot allocate device memory when they call it: a serving
worker bound to the C ABI has no torch allocator to ask, and once it has given the free
HBM to its KV-cache pool a ``cudaMalloc`` would fail or stall the GPU.  For them the library
carries its own 2 MiB scratch buffer.  This test checks that the entry point using that
buffer returns exactly what ``dq_moe_gemv`` returns with caller-provided scratch -- twice in
a row, because the second call finds the first call's leftovers in the shared buffer -- and
that a problem too large for the buffer is refused with a message saying so.

The file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, _lib, ops, x, ids, w, layer, experts, y):
    wgu = ops.weight_descriptor("moe_gemv", layer.gate_up.packed, layer.gate_up.scales, layer.gate_up.offsets,
                                layer.gate_up.bits, 128, layer.gate_up.in_features)
    wdn = ops.weight_descriptor("moe_gemv", layer.down.packed, layer.down.scales, layer.down.offsets,
                                layer.down.bits, 128, layer.down.in_features)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.dq_moe_gemv_static(
        x.data_ptr(), _lib.DQ_BF16, x.shape[0], ids.data_ptr(), w.data_ptr(), ids.shape[1], experts,
        ctypes.byref(wgu), ctypes.byref(wdn), layer.hidden, layer.inter, y.data_ptr(), _lib.DQ_BF16, stream,
    )


def test_static_scratch_entry_point_matches_the_allocating_one_twice():
    from dynquant_b200 import _lib, ops
    from dynquant_b200.workloads import qwen3_moe_layer, seeded_routing

    lib = _lib.load()
    experts, hidden, inter, topk = 32, 1024, 512, 4
    layer = qwen3_moe_layer("cuda", seed=41, bits_gate_up=3, bits_down=4, num_experts=experts, hidden=hidden,
                            inter=inter, topk=topk)
    for call, tokens in enumerate((8, 5)):  # the second call reuses the buffer the first one dirtied
        ids, w = seeded_routing(tokens, experts, topk, seed=100 + call)
        ids, w = ids.cuda(), w.cuda()
        x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(call)).to(torch.bfloat16).cuda()
        want = ops.moe_gemv(x, ids, w, layer.gate_up, layer.down, num_experts=experts)
        got = torch.empty_like(want)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        held_before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        rc = _call_static(lib, _lib, ops, x, ids, w, layer, experts, got)
        assert rc == _lib.DQ_OK, _lib.last_error()
        torch.cuda.synchronize()
        if call > 0:  # (the very first call may load the kernels' code; after that nothing may move)
            # the claim itself: the call obtained no device memory, from the driver or from torch
            assert torch.cuda.mem_get_info()[0] == free_before
            assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == held_before
        # same kernels, same order of operations: bit-identical, not merely close
        assert torch.equal(got, want)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from dynquant_b200 import _lib, ops
    from dynquant_b200.workloads import qwen3_moe_layer, seeded_routing

    lib = _lib.load()
    experts, hidden, inter, topk = 8, 2048, 768, 8
    layer = qwen3_moe_layer("cuda", seed=42, num_experts=experts, hidden=hidden, inter=inter, topk=topk)
    tokens = 64  # 512 assignments x (768 bf16 + 2048 fp32) is ~4.8 MiB of scratch
    assert ops.moe_scratch_bytes(tokens, topk, hidden, inter, experts, torch.bfloat16) > 2 * 1024 * 1024
    ids, w = seeded_routing(tokens, experts, topk)
    x = torch.zeros(tokens, hidden, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(x)
    rc = _call_static(lib, _lib, ops, x, ids.cuda(), w.cuda(), layer, experts, y)
    assert rc == _lib.DQ_ERR_INVALID
    msg = _lib.last_error()
    assert "built-in buffer holds 2097152" in msg and "dq_moe_gemv" in msg
