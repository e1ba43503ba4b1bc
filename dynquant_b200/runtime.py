"""Packed modules: drop-in ``nn.Linear`` / ``nn.Embedding`` replacements over packed weights.

Interface of the reference's ``runtime/linear.py`` -- ``DynQuantLinear(weight, bias=None, *,
tied_to=None)`` with ``from_linear`` and ``forward`` (:174-212), ``DynQuantEmbedding(weight, *,
padding_idx=None, tied_to=None)`` (:215-260), state-dict keys ``qweight`` / ``scales`` /
``offsets`` / ``bias``, an output projection that can borrow the embedding's table, and
``packed_bytes`` -- implemented for a runtime whose only backend is the sm_100a library.

What is different underneath: the reference rebuilds a ``QuantTensor`` view of the buffers on
every forward call (``runtime/linear.py:128-143``) and pays for it in host time per module.
Here the view is built once and kept until the storage under it moves (``.to()``,
``load_state_dict`` with ``assign=True``): a forward is one comparison of a data pointer and
one library call.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from . import ops
from .format import DEFAULT_GROUP_SIZE, QuantTensor

BUFFER_NAMES = ("qweight", "scales", "offsets")  # checkpoint keys of a packed module


@dataclass(frozen=True)
class PackedSpec:
    """Everything about a packed weight that is not a tensor."""

    bits: int
    group_size: int
    in_features: int
    out_features: int
    symmetric: bool
    row_offset: int

    @classmethod
    def of(cls, qt: QuantTensor) -> "PackedSpec":
        if qt.layout != "linear":
            raise NotImplementedError(f"only the linear layout has kernels; this tensor is laid out {qt.layout!r}")
        if len(qt.logical_shape) != 2:
            raise ValueError(f"a packed module holds a matrix; this tensor's logical shape is {qt.logical_shape}")
        return cls(qt.bits, qt.group_size, qt.in_features, qt.num_rows, qt.symmetric, qt.row_offset)

    def view(self, packed: torch.Tensor, scales: torch.Tensor, offsets: torch.Tensor | None) -> QuantTensor:
        return QuantTensor(packed, scales, offsets, self.bits, self.group_size, self.in_features,
                           (self.out_features, self.in_features), row_offset=self.row_offset,
                           symmetric=self.symmetric)


class _PackedModule(nn.Module):
    """Owns the three buffers of one packed matrix -- or borrows another module's.

    A borrowing module (``tied_to=``) registers nothing: the lender is kept outside the module
    tree (so ``state_dict`` holds the table once and ``.to()`` moves it once) and every access
    goes through :attr:`holder`.
    """

    def __init__(self, weight: QuantTensor, *, tied_to: "_PackedModule | None" = None) -> None:
        super().__init__()
        self.spec = PackedSpec.of(weight)
        self.__dict__["_lender"] = tied_to  # bypasses nn.Module.__setattr__: not a child module
        self.__dict__["_view"] = None       # (data_ptr of packed, QuantTensor)
        if tied_to is None:
            for name, tensor in zip(BUFFER_NAMES, (weight.packed, weight.scales, weight.offsets)):
                self.register_buffer(name, tensor)

    # -- the attributes callers of the reference module read --
    bits = property(lambda self: self.spec.bits)
    group_size = property(lambda self: self.spec.group_size)
    in_features = property(lambda self: self.spec.in_features)
    out_features = property(lambda self: self.spec.out_features)
    symmetric = property(lambda self: self.spec.symmetric)
    row_offset = property(lambda self: self.spec.row_offset)

    @property
    def holder(self) -> "_PackedModule":
        lender = self.__dict__["_lender"]
        return self if lender is None else lender.holder

    @property
    def weight_qt(self) -> QuantTensor:
        """The buffers as a ``QuantTensor`` (no copy); rebuilt only when the storage moved."""
        buffers = self.holder._buffers
        packed = buffers[BUFFER_NAMES[0]]
        cached = self.__dict__["_view"]
        if cached is None or cached[0] != packed.data_ptr():
            cached = (packed.data_ptr(), self.spec.view(packed, buffers[BUFFER_NAMES[1]], buffers[BUFFER_NAMES[2]]))
            self.__dict__["_view"] = cached
        return cached[1]

    @property
    def nbytes(self) -> int:
        return self.weight_qt.nbytes

    def extra_repr(self) -> str:
        s = self.spec
        grouping = f"groups of {s.group_size}" if s.group_size > 0 else "one group per row"
        return (f"{s.in_features} -> {s.out_features}, {s.bits}-bit, {grouping}, "
                f"{8.0 * self.nbytes / (s.in_features * s.out_features):.2f} bits per weight stored")


def _encode(weight: torch.Tensor, bits: int, group_size: int, symmetric: bool) -> QuantTensor:
    """Min/max encoding of a dense weight on its own device's host copy (no clip search: the
    reference's encoder search is outside this package)."""
    w = weight.detach()
    meta = w.dtype if w.dtype in (torch.float16, torch.bfloat16) else torch.float16
    qt = QuantTensor.from_dense(w.cpu(), bits=bits, group_size=group_size, symmetric=symmetric, compute_dtype=meta)
    return qt.to(w.device)


class DynQuantLinear(_PackedModule):
    """``y = x @ W.T + b`` with ``W`` packed in HBM; inference only."""

    def __init__(self, weight: QuantTensor, bias: torch.Tensor | None = None, *,
                 tied_to: _PackedModule | None = None) -> None:
        super().__init__(weight, tied_to=tied_to)
        self.register_buffer("bias", bias.detach().clone() if bias is not None else None)

    @classmethod
    def from_linear(cls, linear: nn.Linear, bits: int, *, group_size: int = DEFAULT_GROUP_SIZE,
                    symmetric: bool = False) -> "DynQuantLinear":
        return cls(_encode(linear.weight, bits, group_size, symmetric), linear.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.quantized_matmul(x, self.weight_qt, self.bias)


class DynQuantEmbedding(_PackedModule):
    """Token table stored packed: the looked-up rows are gathered packed, then decoded."""

    def __init__(self, weight: QuantTensor, *, padding_idx: int | None = None,
                 tied_to: _PackedModule | None = None) -> None:
        super().__init__(weight, tied_to=tied_to)
        self.padding_idx = padding_idx

    num_embeddings = property(lambda self: self.spec.out_features)
    embedding_dim = property(lambda self: self.spec.in_features)

    @classmethod
    def from_embedding(cls, embedding: nn.Embedding, bits: int, *, group_size: int = DEFAULT_GROUP_SIZE,
                       symmetric: bool = False) -> "DynQuantEmbedding":
        return cls(_encode(embedding.weight, bits, group_size, symmetric), padding_idx=embedding.padding_idx)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding_lookup(self.weight_qt, ids)


def packed_bytes(module: nn.Module) -> int:
    """Packed bytes resident under ``module``; a table that is lent out counts once."""
    owners = {id(sub.holder): sub.holder for sub in module.modules() if isinstance(sub, _PackedModule)}
    return sum(owner.nbytes for owner in owners.values())
