"""Peer-memory exchanges (``dq_peer_*``): one GPU here, two in ``test_gpu_multi.py``.

On one device a "group" is a list of buffers of this process.  A world of one exercises the
copy, flag and epoch logic over many calls; a world of two whose second rank never launches
makes the bounded wait run out -- the only way a failure is produced here: a flag that nothing
sets.  Nothing faults or hangs: the kernel gives up after its poll budget and reports.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(world, piece_bytes):
    from dynquant_b200 import _lib

    header = int(_lib.load().dq_peer_header_bytes())
    half = -(-piece_bytes * world // 256) * 256
    return [torch.zeros(header + 2 * half, dtype=torch.uint8, device="cuda") for _ in range(world)]


def test_world_of_one_round_trips_many_times():
    from dynquant_b200.peer import PeerExchange

    ex = PeerExchange.from_buffers(_buffers(1, 1 << 19), rank=0)
    for call, n in enumerate((16, 4096, 8, 65536, 131072)):  # sizes from one CTA to eight per peer
        piece = torch.randn(n, device="cuda").to(torch.bfloat16)
        out = torch.empty_like(piece)
        ex.all_gather(piece, out)
        ex.check()
        assert torch.equal(out, piece), call
        partial = torch.randn(n, device="cuda")
        summed = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        ex.reduce_scatter(partial, summed)
        ex.check()
        assert torch.equal(summed, partial.to(torch.bfloat16)), call


def test_a_peer_that_never_answers_makes_the_wait_run_out():
    from dynquant_b200.peer import PeerExchange

    ex = PeerExchange.from_buffers(_buffers(2, 4096), rank=0, spin_limit=2000)
    piece = torch.ones(1024, device="cuda")
    out = torch.zeros(2048, device="cuda")
    ex.all_gather(piece, out)
    with pytest.raises(RuntimeError, match="gave up waiting for the piece of rank 1"):
        ex.check()
    assert torch.equal(out[:1024], piece)  # its own piece arrived; the other slot was left alone
    assert not bool(out[1024:].any())


def test_pieces_that_do_not_fit_are_refused():
    from dynquant_b200.peer import PeerExchange

    ex = PeerExchange.from_buffers(_buffers(1, 1024), rank=0)
    piece = torch.zeros(4096, device="cuda")
    with pytest.raises(RuntimeError, match="per half of the exchange buffer"):
        ex.all_gather(piece, torch.empty_like(piece))
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ex.all_gather(torch.zeros(3, device="cuda"), torch.zeros(3, device="cuda"))


# ---- a stage's all-gather folded into its GEMV launch (dq_gemv_stage_push) ----

def _stage_jobs(weights, x, out, m):
    """A ``dq_gemv_job`` array: every weight reads ``x`` and writes its columns of ``out``."""
    from dynquant_b200 import _lib
    from dynquant_b200.ops import _tag, weight_descriptor

    jobs = (_lib.GemvJob * len(weights))()
    col = 0
    for job, qt in zip(jobs, weights):
        job.x, job.out, job.bias, job.m = x.data_ptr(), out.data_ptr(), None, m
        job.out_stride, job.out_col0 = out.shape[1], col
        job.x_dtype, job.out_dtype = _tag(x.dtype, "x"), _tag(out.dtype, "out")
        job.weight = weight_descriptor("test", qt.packed, qt.scales, qt.offsets, qt.bits, qt.geometry.effective_group,
                                       qt.in_features)
        col += qt.num_rows
    return jobs


def _windows(world, piece_bytes, exchanges=1):
    from dynquant_b200.peer import PushWindow

    need = PushWindow.bytes_needed([piece_bytes] * exchanges, world)
    return [torch.zeros(need, dtype=torch.uint8, device="cuda") for _ in range(world)]


@pytest.mark.parametrize(("shapes", "m", "kernel"), [
    ([(2048, 4), (512, 2), (512, 3)], 1, "gemv_mma_tile_kernel"),   # a fused q/k/v stage, mixed widths
    ([(6144, 3), (6144, 8)], 3, "gemv_mma_tile_kernel"),            # gate/up, three activation rows
    ([(1000, 4)], 2, "gemv_mma_tile_kernel"),                       # a ragged row count: the last item is short
    ([(20480, 8)], 1, "gemv_mma_stream_kernel"),                    # a long matrix: the streaming kernel pushes too
    ([(19001, 4)], 8, "gemv_mma_stream_kernel"),
])
def test_world_of_one_push_equals_the_plain_stage(shapes, m, kernel):
    from dynquant_b200 import _lib, ops
    from dynquant_b200.peer import PushWindow
    from dynquant_b200.workloads import random_quant_tensor

    gen = torch.Generator(device="cuda").manual_seed(11)
    k = 512
    weights = [random_quant_tensor(rows, k, bits, device="cuda", generator=gen) for rows, bits in shapes]
    cols = sum(r for r, _ in shapes)
    x = torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16)
    want = torch.empty(m, cols, dtype=torch.bfloat16, device="cuda")
    jobs = _stage_jobs(weights, x, want, m)
    _lib.check(_lib.load().dq_gemv_sequence(jobs, len(weights), ops._stream(want.device)))
    out = torch.zeros_like(want)
    jobs = _stage_jobs(weights, x, out, m)
    piece_bytes = out.numel() * 2
    win = PushWindow([piece_bytes], buffers=_windows(1, piece_bytes), rank=0)
    for step in range(1, 4):  # epochs 1, 2, 3: halves 1, 0, 1
        out.zero_()
        assert win.run_stage(0, jobs, len(weights))
        assert _lib.load().dq_last_kernel().decode() == kernel
        win.check()
        assert win.epoch(0) == step
        got = win.piece(0)[0, :piece_bytes].view(torch.bfloat16).view(m, cols)
        assert torch.equal(out, want) and torch.equal(got, want), step
    other = win.piece(0, epoch=2)[0, :piece_bytes].view(torch.bfloat16).view(m, cols)
    assert torch.equal(other, want)  # the other half still holds the step before


def test_push_lands_in_every_window_and_a_rank_that_never_answers_is_reported():
    from dynquant_b200 import _lib, ops
    from dynquant_b200.peer import PushWindow
    from dynquant_b200.workloads import random_quant_tensor

    gen = torch.Generator(device="cuda").manual_seed(12)
    weights = [random_quant_tensor(1024, 256, 4, device="cuda", generator=gen),
               random_quant_tensor(256, 256, 2, device="cuda", generator=gen)]
    x = torch.randn(2, 256, device="cuda", generator=gen).to(torch.bfloat16)
    out = torch.zeros(2, 1280, dtype=torch.bfloat16, device="cuda")
    jobs = _stage_jobs(weights, x, out, 2)
    piece_bytes = out.numel() * 2
    buffers = _windows(3, piece_bytes)
    # this process plays rank 1 of 3; rank 0 "has answered" (its flag is already far ahead), rank 2 never does
    win = PushWindow([piece_bytes], buffers=buffers, rank=1, spin_limit=2000)
    flags = buffers[1][win._HEAD + 64:win._HEAD + 64 + 12].view(torch.int32)
    flags[0] = 1000
    assert win.run_stage(0, jobs, 2)
    with pytest.raises(RuntimeError, match="gave up waiting for the rows of rank 2"):
        win.check()
    want = torch.empty_like(out)
    _lib.check(_lib.load().dq_gemv_sequence(_stage_jobs(weights, x, want, 2), 2, ops._stream(out.device)))
    torch.cuda.synchronize()
    for r in range(3):  # rank 1's slot of half 1 (epoch 1) in every window; the other slots untouched
        data = buffers[r][win._data_off[0]:win._data_off[0] + 2 * 3 * piece_bytes].view(2, 3, piece_bytes)
        assert torch.equal(data[1, 1].view(torch.bfloat16).view(2, 1280), want), r
        assert not bool(data[0].any()) and not bool(data[1, 0].any()) and not bool(data[1, 2].any()), r
        assert int(buffers[r][win._HEAD + 64 + 4:win._HEAD + 64 + 8].view(torch.int32).item()) == 1  # rank 1's flag
    # the context is still usable and the next launch does not spin again: the status word is set
    assert win.run_stage(0, jobs, 2)
    torch.cuda.synchronize()


def test_stages_the_pushing_kernels_do_not_take_are_refused_without_a_launch():
    from dynquant_b200 import _lib
    from dynquant_b200.peer import PushWindow
    from dynquant_b200.workloads import random_quant_tensor

    gen = torch.Generator(device="cuda").manual_seed(13)
    qt = random_quant_tensor(64, 100, 4, group_size=-1, device="cuda", generator=gen)  # per-row groups: SIMT only
    x = torch.randn(1, 100, device="cuda", generator=gen).to(torch.bfloat16)
    out = torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda")
    win = PushWindow([128], buffers=_windows(1, 128), rank=0)
    before = int(_lib.load().dq_launch_count())
    assert not win.run_stage(0, _stage_jobs([qt], x, out, 1), 1)
    assert int(_lib.load().dq_launch_count()) == before
    assert win.epoch(0) == 0


def test_world_of_one_gathers_several_tensors_in_one_launch():
    from dynquant_b200 import _lib
    from dynquant_b200.peer import PeerExchange

    ex = PeerExchange.from_buffers(_buffers(1, 1 << 19), rank=0)
    for sizes in ((4096, 32, 32), (16, 16), (131072, 64, 48, 16)):  # the last: several CTAs, a part inside one CTA's span
        pieces = [torch.randint(0, 255, (n,), dtype=torch.uint8, device="cuda") for n in sizes]
        outs = [torch.zeros_like(p) for p in pieces]
        before = int(_lib.load().dq_launch_count())
        ex.all_gather_parts(pieces, outs)
        assert int(_lib.load().dq_launch_count()) - before == 1
        ex.check()
        assert all(torch.equal(o, p) for o, p in zip(outs, pieces)), sizes
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ex.all_gather_parts([torch.zeros(24, dtype=torch.uint8, device="cuda")], [torch.zeros(24, dtype=torch.uint8, device="cuda")])
