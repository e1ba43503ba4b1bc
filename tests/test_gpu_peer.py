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
