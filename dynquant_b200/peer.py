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

    def all_gather_parts(self, pieces: list[torch.Tensor], outs: list[torch.Tensor]) -> list[torch.Tensor]:
        """Up to four tensors in ONE exchange launch: ``outs[i]`` (``world`` times ``pieces[i]``)
        receives every rank's ``pieces[i]`` in rank order."""
        n = len(pieces)
        sizes = [p.numel() * p.element_size() for p in pieces]
        for p, o, b in zip(pieces, outs, sizes):
            if not p.is_contiguous() or not o.is_contiguous() or o.numel() * o.element_size() != b * self.world:
                raise RuntimeError("peer all_gather_parts: pieces and outs must be contiguous and outs hold world pieces")
        srcs = (ctypes.c_void_p * n)(*[p.data_ptr() for p in pieces])
        dsts = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outs])
        nbytes = (ctypes.c_int64 * n)(*sizes)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().dq_peer_all_gather_parts(ctypes.byref(self._desc), srcs, nbytes, dsts, n,
                                                            _stream(self.device)))
        return outs

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


class PushWindow:
    """One window per rank for stages whose all-gather is folded into the GEMV launch
    (``dq_gemv_stage_push``): the producing kernel stores its output rows into every rank's
    window and ends with a bounded wait for the other ranks' rows.

    ``piece_bytes[i]`` is the size of exchange ``i``'s piece (one rank's ``[m, columns]`` output
    buffer).  Layout of a window, identical on every rank: the status word, then per exchange 64
    bytes of state and 64 of flags, then per exchange two halves of ``world`` pieces.
    ``piece(i, epoch)`` views what exchange ``i`` gathered as ``[world, piece_bytes]`` bytes.
    """

    _SLOT = 128   # per exchange: u32[2] state at +0, u32[world <= 8] flags at +64
    _HEAD = 256   # the status word and padding

    def __init__(self, piece_bytes: list[int], *, group=None, device=None, spin_limit: int = 0,
                 buffers: list[torch.Tensor] | None = None, rank: int | None = None) -> None:
        self.pieces = [-(-int(b) // 16) * 16 for b in piece_bytes]
        self.spin_limit = spin_limit
        table_bytes = self._HEAD + self._SLOT * len(self.pieces)
        table_bytes = -(-table_bytes // 256) * 256
        self._data_off = []
        at = table_bytes
        world = len(buffers) if buffers is not None else None
        if buffers is None:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm

            group = group if group is not None else dist.group.WORLD
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            world = self.world
        else:
            self.world, self.rank = world, int(rank)
        if self.world > 8:
            raise RuntimeError(f"a push window serves at most 8 ranks, got {self.world}")
        for b in self.pieces:
            self._data_off.append(at)
            at += -(-2 * world * b // 256) * 256
        self.window_bytes = at
        if buffers is None:
            self.device = torch.device(device if device is not None else ("cuda", torch.cuda.current_device()))
            self.buffer = symm.empty(self.window_bytes, dtype=torch.uint8, device=self.device)
            self.buffer.zero_()
            self.handle = symm.rendezvous(self.buffer, group=group)
            torch.cuda.synchronize(self.device)
            dist.barrier(group)  # every window is zero before anyone stores into a peer's
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
        else:
            # windows of THIS process (tests: a world of one, or peers that never answer)
            if any(b.numel() < self.window_bytes for b in buffers):
                raise RuntimeError(f"every window needs {self.window_bytes} bytes")
            self.device = buffers[0].device
            self._buffers = list(buffers)
            self.buffer = buffers[self.rank]
            self.handle = None
            ptrs = [b.data_ptr() for b in buffers]
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        self._descs = [
            _lib.PeerPush(self._ptrs, self.world, self.rank, self._data_off[i], self.pieces[i],
                          self._HEAD + self._SLOT * i + 64, self._HEAD + self._SLOT * i, 0, spin_limit, 0)
            for i in range(len(self.pieces))
        ]

    @staticmethod
    def bytes_needed(piece_bytes: list[int], world: int) -> int:
        table = -(-(PushWindow._HEAD + PushWindow._SLOT * len(piece_bytes)) // 256) * 256
        return table + sum(-(-2 * world * (-(-int(b) // 16) * 16) // 256) * 256 for b in piece_bytes)

    def run_stage(self, index: int, jobs, count: int) -> bool:
        """Enqueue exchange ``index``'s stage (``count`` jobs of a ``dq_gemv_job`` array).  False,
        with nothing launched, when the jobs do not leave as one pushing launch."""
        lib = _lib.load()
        with torch.cuda.device(self.device):
            rc = lib.dq_gemv_stage_push(jobs, count, ctypes.byref(self._descs[index]), _stream(self.device))
        if rc == _lib.DQ_ERR_UNSUPPORTED:
            return False
        _lib.check(rc)
        return True

    def epoch(self, index: int) -> int:
        """Exchanges ``index`` has completed (synchronises)."""
        torch.cuda.synchronize(self.device)
        at = self._HEAD + self._SLOT * index
        return int(self.buffer[at:at + 4].view(torch.int32).item())

    def piece(self, index: int, epoch: int | None = None) -> torch.Tensor:
        """``[world, piece_bytes]`` bytes: what exchange ``index`` gathered at ``epoch`` (default:
        its last one)."""
        epoch = self.epoch(index) if epoch is None else epoch
        b = self.pieces[index]
        at = self._data_off[index] + (epoch & 1) * self.world * b
        return self.buffer[at:at + self.world * b].view(self.world, b)

    def check(self) -> None:
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().dq_peer_push_status(ctypes.byref(self._descs[0]), _stream(self.device)))
