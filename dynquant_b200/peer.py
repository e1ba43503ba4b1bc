"""Exchanges of the sharded paths over peer memory (``dq_peer_*`` of the C ABI).

:class:`PeerExchange` owns one exchange buffer per rank, mapped into every rank of a process
group (``torch.distributed._symmetric_memory``: CUDA virtual-memory handles passed between the
processes of one node), and offers the two exchanges the sharded paths need -- an all-gather of
small output slabs and a reduce-scatter of fp32 partial rows -- as ordinary kernel launches on
torch's current stream.  They can be captured in the CUDA graph of a decode step, which a
host-issued collective per module cannot without every rank capturing in lock step.

All ranks must call the same sequence of exchanges.  ``check()`` synchronises and raises if a
wait for a peer's piece ran out of polls (a peer that never launched, or died).
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .ops import _stream, _tag


class PeerExchange:
    def __init__(self, max_piece_bytes: int, *, group=None, device=None, spin_limit: int = 0) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device if device is not None else ("cuda", torch.cuda.current_device()))
        header = int(_lib.load().dq_peer_header_bytes())
        half = -(-max_piece_bytes * self.world // 256) * 256
        self.buffer_bytes = header + 2 * half
        self.buffer = symm.empty(self.buffer_bytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        self.handle = symm.rendezvous(self.buffer, group=group)
        torch.cuda.synchronize(self.device)
        dist.barrier(group)  # every buffer is zero before anyone stores into a peer's
        self._desc = _lib.PeerGroup(int(self.handle.buffer_ptrs_dev), self.buffer_bytes, self.world, self.rank,
                                    spin_limit, 0)

    @classmethod
    def from_buffers(cls, buffers: list[torch.Tensor], rank: int, spin_limit: int = 0) -> "PeerExchange":
        """A group over buffers of THIS process (tests: a world of one, or a peer that never
        answers).  ``buffers[i]`` stands for rank i's exchange buffer."""
        self = cls.__new__(cls)
        self.world, self.rank = len(buffers), rank
        self.device = buffers[0].device
        self._buffers = list(buffers)  # every "rank's" buffer stays alive as long as the group does
        self.buffer = buffers[rank]
        self.buffer_bytes = buffers[0].numel()
        self._table = torch.tensor([b.data_ptr() for b in buffers], dtype=torch.int64, device=self.device)
        self.handle = None
        self._desc = _lib.PeerGroup(self._table.data_ptr(), self.buffer_bytes, self.world, rank, spin_limit, 0)
        return self

    def all_gather(self, piece: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``out`` (``world`` times the size of ``piece``, contiguous) receives every rank's piece
        in rank order."""
        nbytes = piece.numel() * piece.element_size()
        if not piece.is_contiguous() or not out.is_contiguous() or out.numel() * out.element_size() != nbytes * self.world:
            raise RuntimeError("peer all_gather: piece and out must be contiguous and out must hold world pieces")
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().dq_peer_all_gather(ctypes.byref(self._desc), piece.data_ptr(), nbytes, out.data_ptr(),
                                                      _stream(self.device)))
        return out

    def reduce_scatter(self, partial: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``partial``: fp32 ``[world * n]`` (rank i's rows first-to-last at ``[i * n, (i + 1) * n)``);
        ``out``: ``n`` elements receiving the sum over source ranks of this rank's rows."""
        if partial.dtype != torch.float32 or not partial.is_contiguous() or not out.is_contiguous():
            raise RuntimeError("peer reduce_scatter: partial must be contiguous float32 and out contiguous")
        if partial.numel() != out.numel() * self.world:
            raise RuntimeError("peer reduce_scatter: partial must hold world times the elements of out")
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().dq_peer_reduce_scatter_f32(ctypes.byref(self._desc), partial.data_ptr(), out.numel(),
                                                              out.data_ptr(), _tag(out.dtype, "out"), _stream(self.device)))
        return out

    def check(self) -> None:
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().dq_peer_status(ctypes.byref(self._desc), self.buffer.data_ptr(), _stream(self.device)))
