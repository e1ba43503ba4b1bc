"""Whole-step plans (``dq_plan_*``): one persistent kernel over a job list.

The oracle is the same as for single GEMVs (``x.float() @ dequant(fp32).T``, 1e-3 on the fp32
accumulators); on top of that a plan must agree with ``dq_gemv_sequence`` over the same jobs,
respect the order of the list when a job reads what the job before it wrote, repeat bit for
bit, and fail cleanly -- status word, ``RuntimeError`` -- when a stage's bounded wait runs out.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from conftest import make_quant
from test_gpu_parity import oracle_gemv

pytestmark = pytest.mark.gpu


def _jobs(entries, m, act_dtype, out_dtype):
    """entries: list of (x tensor, QuantTensor, out tensor) -> ctypes job array."""
    from dynquant_b200 import _lib
    from dynquant_b200.ops import _tag, weight_descriptor

    arr = (_lib.GemvJob * len(entries))()
    for job, (x, qt, out) in zip(arr, entries):
        job.x, job.out, job.bias = x.data_ptr(), out.data_ptr(), None
        job.m, job.out_stride, job.out_col0 = m, out.shape[1], 0
        job.x_dtype, job.out_dtype = _tag(act_dtype, "x"), _tag(out_dtype, "out")
        job.weight = weight_descriptor("plan", qt.packed, qt.scales, qt.offsets, qt.bits,
                                       qt.geometry.effective_group, qt.in_features)
    return arr


def _close(got: torch.Tensor, want: np.ndarray, tol=1e-3):
    g = got.float().cpu().numpy()
    scale = np.abs(want).max() + 1e-30
    assert np.abs(g - want).max() / scale <= tol
    assert np.linalg.norm(g - want) / (np.linalg.norm(want) + 1e-30) <= tol


@pytest.mark.parametrize("m", [1, 3, 8])
def test_plan_matches_the_oracle_and_the_sequence_call(m):
    """Two decoder layers of the benchmark stack's shapes plus a 4,000-row head (every width,
    fused q/k/v and gate/up stages, a 48-step reduction, a row count that is not a multiple of
    16): every module against the CPU oracle, and against dq_gemv_sequence."""
    from dynquant_b200 import _lib
    from dynquant_b200.stack import GemvPlan
    from dynquant_b200.ops import _stream

    dev = torch.device("cuda")
    hidden, inter = 2048, 6144
    shapes = [("q", 2048, hidden, "h", 4), ("k", 1024, hidden, "h", 2), ("v", 1024, hidden, "h", 3),
              ("o", 2048, 2048, "a", 8), ("gate", inter, hidden, "h", 3), ("up", inter, hidden, "h", 2),
              ("down", hidden, inter, "i", 4),
              ("q2", 2048, hidden, "h", 3), ("k2", 1024, hidden, "h", 8), ("v2", 1024, hidden, "h", 4),
              ("o2", 2048, 2048, "a", 2), ("gate2", inter, hidden, "h", 4), ("up2", inter, hidden, "h", 8),
              ("down2", hidden, inter, "i", 3), ("head", 4001, hidden, "h", 8)]
    gen = torch.Generator().manual_seed(100 + m)
    acts = {"h": torch.randn(m, hidden, generator=gen), "a": torch.randn(m, 2048, generator=gen),
            "i": torch.randn(m, inter, generator=gen)}
    acts = {k: v.to(torch.bfloat16).to(dev) for k, v in acts.items()}
    entries, entries_seq = [], []
    for idx, (name, rows, k, src, bits) in enumerate(shapes):
        qt = make_quant(rows, k, 128, bits, torch.float16, seed=500 + idx).to(dev)
        entries.append((acts[src], qt, torch.full((m, rows), float("nan"), dtype=torch.float32, device=dev)))
        entries_seq.append((acts[src], qt, torch.empty((m, rows), dtype=torch.float32, device=dev)))
    jobs = _jobs(entries, m, torch.bfloat16, torch.float32)
    plan = GemvPlan(jobs, len(entries), dev)
    info = plan.info()
    assert info["num_jobs"] == len(shapes) and info["num_stages"] == 9  # qkv, o, gate/up, down, twice, head
    before = _lib.load().dq_launch_count()
    plan.launch()
    assert _lib.load().dq_launch_count() - before == 1
    plan.check()
    seq = _jobs(entries_seq, m, torch.bfloat16, torch.float32)
    _lib.check(_lib.load().dq_gemv_sequence(seq, len(entries_seq), _stream(dev)))
    torch.cuda.synchronize()
    for (x, qt, out), (_, _, out_seq) in zip(entries, entries_seq):
        want = oracle_gemv(x, qt)
        _close(out, want)
        assert np.abs(out.cpu().numpy() - out_seq.cpu().numpy()).max() / np.abs(want).max() <= 2e-5
    first = [out.clone() for _, _, out in entries]
    for _ in range(5):  # replays are bit-identical (fixed summation order, counters reset themselves)
        for _, _, out in entries:
            out.fill_(float("nan"))
        plan.launch()
        plan.check()
        for (_, _, out), ref in zip(entries, first):
            assert torch.equal(out, ref)
    plan.close()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_plan_orders_jobs_that_feed_each_other(dtype):
    """A true chain -- every job reads the 16-bit output of the job before it -- replayed many
    times: a stage that read its activation before the previous stage had stored it would
    disagree with the same chain run as separate, stream-ordered launches."""
    from dynquant_b200 import ops
    from dynquant_b200.stack import GemvPlan

    dev = torch.device("cuda")
    m = 2
    dims = [1024, 2048, 512, 6144, 1024, 256, 2048, 1024]
    bits = [4, 2, 3, 8, 2, 4, 3]
    meta = torch.float16 if dtype == torch.bfloat16 else torch.bfloat16
    qts = [make_quant(dims[i + 1], dims[i], 128, bits[i], meta, seed=900 + i).to(dev) for i in range(len(bits))]
    # keep the chain's magnitude near 1: scale every layer by 1/sqrt(K)
    for i, qt in enumerate(qts):
        qt.scales.mul_(1.0 / dims[i] ** 0.5)
        if qt.offsets is not None:
            qt.offsets.mul_(1.0 / dims[i] ** 0.5)
    x0 = torch.randn(m, dims[0], generator=torch.Generator().manual_seed(3)).to(dtype).to(dev)
    bufs = [x0] + [torch.zeros(m, d, dtype=dtype, device=dev) for d in dims[1:]]
    entries = [(bufs[i], qts[i], bufs[i + 1]) for i in range(len(qts))]
    plan = GemvPlan(_jobs(entries, m, dtype, dtype), len(entries), dev)
    assert plan.info()["num_stages"] == len(qts)
    # the same chain, one launch per link
    want = x0
    for qt in qts:
        want = ops.gemv(want, qt.packed, qt.scales, qt.offsets, qt.bits, 128, qt.in_features)
    torch.cuda.synchronize()
    for rep in range(20):
        for b in bufs[1:]:
            b.zero_()
        plan.launch()
        plan.check()
        # slicing differs between the two kernels, so intermediate roundings may differ in the last bit
        err = (bufs[-1].float() - want.float()).abs().max().item() / (want.float().abs().max().item() + 1e-30)
        assert err <= 2e-2, (rep, err)
        if rep == 0:
            first = [b.clone() for b in bufs[1:]]
        else:
            assert all(torch.equal(b, f) for b, f in zip(bufs[1:], first))
    plan.close()


def test_plan_wait_that_cannot_be_satisfied_runs_out_and_reports():
    """Stage 2 is told to wait for more arrivals than stage 1 has CTAs: its bounded spin runs
    out, the kernel returns, the status call raises, and the plan works again afterwards."""
    from dynquant_b200.stack import GemvPlan

    dev = torch.device("cuda")
    m = 1
    qts = [make_quant(512, 512, 128, b, torch.float16, seed=70 + b).to(dev) for b in (4, 3, 2)]
    x = torch.randn(m, 512, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).to(dev)
    bufs = [x] + [torch.zeros(m, 512, dtype=torch.bfloat16, device=dev) for _ in qts]
    entries = [(bufs[i], qts[i], bufs[i + 1]) for i in range(3)]
    plan = GemvPlan(_jobs(entries, m, torch.bfloat16, torch.bfloat16), 3, dev)
    plan.launch()
    plan.check()
    good = bufs[-1].clone()
    plan.set_wait(2, 1_000_000, 2000)  # no stage has a million CTAs
    plan.launch()
    with pytest.raises(RuntimeError, match="gave up waiting"):
        plan.check()
    # a later healthy launch is unaffected: counters and status were cleared by the check
    grid = plan.info()["grid"]
    shape = plan.stage_shape(1)
    plan.set_wait(2, sum(shape["ctas"]), 1 << 21)
    assert sum(shape["ctas"]) <= grid
    bufs[-1].zero_()
    plan.launch()
    plan.check()
    assert torch.equal(bufs[-1], good)
    plan.close()


def test_plan_refuses_what_the_kernel_cannot_run():
    from dynquant_b200.stack import GemvPlan

    dev = torch.device("cuda")
    x = torch.randn(1, 1024, dtype=torch.bfloat16, device=dev)
    qt = make_quant(64, 1024, 64, 4, torch.float16).to(dev)  # 64-value groups
    out = torch.empty(1, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="dq_gemv_sequence"):
        GemvPlan(_jobs([(x, qt, out)], 1, torch.bfloat16, torch.bfloat16), 1, dev)
    x9 = torch.randn(9, 1024, dtype=torch.bfloat16, device=dev)
    qt2 = make_quant(64, 1024, 128, 4, torch.float16).to(dev)
    out9 = torch.empty(9, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="exceeds the kernel's limit"):
        GemvPlan(_jobs([(x9, qt2, out9)], 9, torch.bfloat16, torch.bfloat16), 1, dev)


def test_step_runner_plan_mode_matches_dataflow_mode():
    """The benchmark's runner: the step as one captured plan kernel against the launch-per-stage
    graph, on a reduced stack with a long 8-bit head (the streaming regime inside the plan)."""
    from dynquant_b200.stack import StepRunner
    from dynquant_b200.workloads import qwen2b_stack

    dev = torch.device("cuda")
    stack = qwen2b_stack(device=dev, vocab=40000, layers=2)
    a = StepRunner(stack, 1, device=dev, out_dtype=torch.float32)
    b = StepRunner(stack, 1, device=dev, out_dtype=torch.float32)
    for k in a.inputs:
        b.inputs[k].copy_(a.inputs[k])
    a.capture("plan")
    # one persistent kernel for the decoder layers, the 40,000-row head on the streaming kernel
    assert a.launches_per_step == 2 and a.plan().info()["launches"] == 2
    b.capture("dataflow")
    a.replay()
    b.replay()
    a.plan().check()
    torch.cuda.synchronize()
    for mod in stack.modules:
        pa, pb = a.outputs[mod.name], b.outputs[mod.name]
        scale = pb.abs().max().item() + 1e-30
        assert (pa - pb).abs().max().item() / scale <= 2e-5, mod.name
