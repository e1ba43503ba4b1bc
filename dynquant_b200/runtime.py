"""Packed modules: ``nn.Linear`` / ``nn.Embedding`` whose weights stay packed in HBM.

Host-side mirror of the reference's ``runtime/linear.py`` (``_PackedModule`` :68-143,
``DynQuantLinear`` :174-212, ``DynQuantEmbedding`` :215-260): same constructor signatures,
same buffer names (``qweight`` / ``scales`` / ``offsets`` / ``bias``), same tied-table
handling, same forward semantics.  The forward calls go to the sm_100a kernels through
:mod:`dynquant_b200.ops`; there is no other backend.
"""

from __future__ import annotations

import torch
from torch import nn

from . import ops
from .format import DEFAULT_GROUP_SIZE, QuantTensor

_PACKED, _SCALES, _OFFSETS = "qweight", "scales", "offsets"


class _PackedModule(nn.Module):
    """Shared storage and plumbing for the two packed module types."""

    def __init__(self, weight: QuantTensor, *, tied_to: "_PackedModule | None" = None) -> None:
        super().__init__()
        if weight.layout != "linear":
            raise NotImplementedError(f"layout {weight.layout} is not runnable yet")
        if len(weight.logical_shape) != 2:
            raise ValueError(f"expected a 2-D weight, got {weight.logical_shape}")
        if tied_to is None:
            self.register_buffer(_PACKED, weight.packed)
            self.register_buffer(_SCALES, weight.scales)
            self.register_buffer(_OFFSETS, weight.offsets)
        else:
            # not a submodule: the tied module only borrows the holder's buffers
            object.__setattr__(self, "_tied_to", tied_to)
        self.bits = weight.bits
        self.group_size = weight.group_size
        self.in_features = weight.in_features
        self.out_features = weight.num_rows
        self.symmetric = weight.symmetric
        self.row_offset = weight.row_offset

    @property
    def holder(self) -> "_PackedModule":
        """The module the buffers live on: this one, or the one it is tied to."""
        return self.__dict__.get("_tied_to", self)

    @property
    def weight_qt(self) -> QuantTensor:
        """A view of this module's buffers as a QuantTensor.  Copies nothing."""
        holder = self.holder
        return QuantTensor(
            packed=holder.get_buffer(_PACKED),
            scales=holder.get_buffer(_SCALES),
            offsets=getattr(holder, _OFFSETS),
            bits=self.bits,
            group_size=self.group_size,
            in_features=self.in_features,
            logical_shape=(self.out_features, self.in_features),
            row_offset=self.row_offset,
            symmetric=self.symmetric,
        )

    @property
    def nbytes(self) -> int:
        return self.weight_qt.nbytes

    def extra_repr(self) -> str:
        group = "per-row" if self.group_size < 0 else f"g{self.group_size}"
        bpw = self.nbytes * 8.0 / (self.in_features * self.out_features)
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"{group}, {bpw:.2f} bits/weight")


class DynQuantLinear(_PackedModule):
    """``nn.Linear`` whose weight lives packed.  Forward only."""

    bias: torch.Tensor | None

    def __init__(self, weight: QuantTensor, bias: torch.Tensor | None = None, *,
                 tied_to: _PackedModule | None = None) -> None:
        super().__init__(weight, tied_to=tied_to)
        self.register_buffer("bias", None if bias is None else bias.detach().clone())

    @classmethod
    def from_linear(cls, linear: nn.Linear, bits: int, *, group_size: int = DEFAULT_GROUP_SIZE,
                    symmetric: bool = False) -> "DynQuantLinear":
        """Plain min/max quantization of ``linear.weight`` (the reference's clip search is an
        encoder feature outside this package's scope)."""
        w = linear.weight.detach()
        dtype = w.dtype if w.dtype in (torch.float16, torch.bfloat16) else torch.float16
        qt = QuantTensor.from_dense(w.cpu(), bits=bits, group_size=group_size, symmetric=symmetric,
                                    compute_dtype=dtype)
        return cls(qt.to(w.device), linear.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.quantized_matmul(x, self.weight_qt, self.bias)


class DynQuantEmbedding(_PackedModule):
    """``nn.Embedding`` whose table lives packed: rows are gathered packed, then dequantized."""

    def __init__(self, weight: QuantTensor, *, padding_idx: int | None = None,
                 tied_to: _PackedModule | None = None) -> None:
        super().__init__(weight, tied_to=tied_to)
        self.padding_idx = padding_idx
        self.num_embeddings = self.out_features
        self.embedding_dim = self.in_features

    @classmethod
    def from_embedding(cls, embedding: nn.Embedding, bits: int, *, group_size: int = DEFAULT_GROUP_SIZE,
                       symmetric: bool = False) -> "DynQuantEmbedding":
        w = embedding.weight.detach()
        dtype = w.dtype if w.dtype in (torch.float16, torch.bfloat16) else torch.float16
        qt = QuantTensor.from_dense(w.cpu(), bits=bits, group_size=group_size, symmetric=symmetric,
                                    compute_dtype=dtype)
        return cls(qt.to(w.device), padding_idx=embedding.padding_idx)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding_lookup(self.weight_qt, ids)


def packed_bytes(module: nn.Module) -> int:
    """Bytes of packed weight resident under ``module``, tied tables counted once."""
    seen: set[int] = set()
    total = 0
    for sub in module.modules():
        if isinstance(sub, _PackedModule):
            holder = sub.holder
            if id(holder) not in seen:
                seen.add(id(holder))
                total += holder.nbytes
    return total
