"""The packed-weight format: geometry, bit packing and the ``QuantTensor`` container.

Host-side mirror of the reference's format layer
(``packages/dynquant-core/src/dynquant/quant/pack.py:203-402`` and
``quant/tensor.py:119-426``; layout of ``docs/format-spec.md`` sections 3-4):

* ``w ~= q * scale + offset`` with ``q`` an unsigned ``bits``-wide code, one
  ``(scale, offset)`` pair per ``(row, group)``; ``offsets=None`` means zero.
* codes are packed per row, per group, LSB-first into int32 words; a group is a
  whole number of words (``group_size % 32 == 0``) except in per-row mode
  (``group_size == -1``), where the single group rounds up to whole words.

This module only *builds and describes* packed tensors (tests, synthetic
workloads, module construction).  It never stands in for the kernels:
``QuantTensor.dequantize`` and every matmul go through the compiled library.
"""

from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, NamedTuple

import torch

BIT_OPTIONS = (2, 3, 4, 8)
PER_ROW_GROUP_SIZE = -1
DEFAULT_GROUP_SIZE = 128
GROUP_SIZE_ALIGNMENT = 32
COMPUTE_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


class PackingError(ValueError):
    """A tensor, width or group size the format cannot represent."""


class RowGeometry(NamedTuple):
    group_size: int  # as stored: may be the -1 sentinel
    effective_group: int  # values per group for arithmetic
    padded_in_features: int
    num_groups: int
    words_per_group: int

    @property
    def words_per_row(self) -> int:
        return self.num_groups * self.words_per_group

    @property
    def is_per_row(self) -> bool:
        return self.group_size == PER_ROW_GROUP_SIZE


def words_for(bits: int, num_values: int) -> int:
    return -(-num_values * bits // 32)


def row_geometry(bits: int, group_size: int, in_features: int) -> RowGeometry:
    """Every derived size of one packed row; validates as a side effect."""
    if bits not in BIT_OPTIONS:
        raise PackingError(f"bits={bits} not supported; expected one of {list(BIT_OPTIONS)}")
    if in_features <= 0:
        raise PackingError(f"in_features must be positive, got {in_features}")
    if group_size == PER_ROW_GROUP_SIZE:
        return RowGeometry(PER_ROW_GROUP_SIZE, in_features, in_features, 1, words_for(bits, in_features))
    if group_size <= 0 or group_size % GROUP_SIZE_ALIGNMENT != 0:
        raise PackingError(
            f"group_size={group_size} must be a positive multiple of {GROUP_SIZE_ALIGNMENT} "
            f"(or {PER_ROW_GROUP_SIZE} for one group per row)"
        )
    groups = -(-in_features // group_size)
    return RowGeometry(group_size, group_size, groups * group_size, groups, group_size * bits // 32)


# --------------------------------------------------------------------------
# bit packing
# --------------------------------------------------------------------------


def _as_int32(words: torch.Tensor) -> torch.Tensor:
    """int64 values in [0, 2**32) -> the int32 with the same bit pattern."""
    words = words & 0xFFFFFFFF
    return (words - ((words >> 31) << 32)).to(torch.int32)


def pack_nbit(q: torch.Tensor, bits: int, *, validate: bool = True) -> torch.Tensor:
    """Pack codes along the last dim, LSB-first, into int32 words.

    Value ``i`` lands at bits ``[i*bits, i*bits+bits)`` of the row's bit
    string; a trailing partial word is zero-filled.
    """
    if bits not in BIT_OPTIONS:
        raise PackingError(f"bits={bits} not supported; expected one of {list(BIT_OPTIONS)}")
    if q.ndim == 0:
        raise PackingError("cannot pack a 0-dim tensor")
    n = q.shape[-1]
    lead = q.shape[:-1]
    if n == 0:
        return torch.zeros((*lead, 0), dtype=torch.int32, device=q.device)
    qi = q.to(torch.int64)
    if validate:
        lo, hi = int(qi.min()), int(qi.max())
        if lo < 0 or hi >= (1 << bits):
            raise PackingError(
                f"codes out of range for {bits}-bit packing: found [{lo}, {hi}], "
                f"need [0, {(1 << bits) - 1}]"
            )
    nwords = words_for(bits, n)
    if 32 % bits == 0:
        per = 32 // bits
        pad = nwords * per - n
        if pad:
            qi = torch.nn.functional.pad(qi, (0, pad))
        shifts = torch.arange(per, device=q.device, dtype=torch.int64) * bits
        words = (qi.reshape(*lead, nwords, per) << shifts).sum(-1)
        return _as_int32(words)
    # 3-bit: 32 values fill exactly three words; work on those 96-bit blocks.
    blocks = -(-n // 32)
    pad = blocks * 32 - n
    if pad:
        qi = torch.nn.functional.pad(qi, (0, pad))
    v = qi.reshape(*lead, blocks, 32)
    pos = torch.arange(32, device=q.device, dtype=torch.int64) * 3
    out = []
    for w in range(3):
        rel = pos - 32 * w  # where each value starts relative to this word
        left = (v << rel.clamp(min=0, max=31)) * ((rel >= 0) & (rel < 32))
        right = (v >> (-rel).clamp(min=0, max=3)) * ((rel < 0) & (rel > -3))  # straddle spill
        out.append(((left + right) & 0xFFFFFFFF).sum(-1) & 0xFFFFFFFF)
    words = torch.stack(out, dim=-1).reshape(*lead, blocks * 3)[..., :nwords]
    return _as_int32(words)


def unpack_nbit(packed: torch.Tensor, bits: int, num_values: int) -> torch.Tensor:
    """Inverse of :func:`pack_nbit`; uint8 codes ``[..., num_values]``."""
    if bits not in BIT_OPTIONS:
        raise PackingError(f"bits={bits} not supported; expected one of {list(BIT_OPTIONS)}")
    expected = words_for(bits, num_values)
    if packed.shape[-1] != expected:
        raise PackingError(
            f"packed last dim is {packed.shape[-1]}, expected {expected} words for "
            f"{num_values} values at {bits}-bit"
        )
    lead = packed.shape[:-1]
    if num_values == 0:
        return torch.zeros((*lead, 0), dtype=torch.uint8, device=packed.device)
    w = packed.to(torch.int64) & 0xFFFFFFFF
    w = torch.nn.functional.pad(w, (0, 1))
    bit = torch.arange(num_values, device=packed.device, dtype=torch.int64) * bits
    idx = bit >> 5
    both = w[..., idx] | ((w[..., idx + 1] & 0xFF) << 32)
    return ((both >> (bit & 31)) & ((1 << bits) - 1)).to(torch.uint8)


# --------------------------------------------------------------------------
# QuantTensor
# --------------------------------------------------------------------------


@dataclass
class QuantTensor:
    """A group-wise affine-quantized matrix in packed form.

    Field names, meanings and defaults follow the reference container
    (``quant/tensor.py:119-157``) so call sites read the same.
    """

    packed: torch.Tensor  # int32 [rows, words_per_row]
    scales: torch.Tensor  # [rows, num_groups]
    offsets: torch.Tensor | None
    bits: int
    group_size: int
    in_features: int
    logical_shape: tuple[int, ...]
    row_offset: int = 0
    layout: str = "linear"
    symmetric: bool = False
    extra: dict[str, Any] = field(default_factory=dict)

    @property
    def num_rows(self) -> int:
        return int(self.packed.shape[0])

    @property
    def geometry(self) -> RowGeometry:
        return row_geometry(self.bits, self.group_size, self.in_features)

    @property
    def num_groups(self) -> int:
        return self.geometry.num_groups

    @property
    def words_per_group(self) -> int:
        return self.geometry.words_per_group

    @property
    def padded_in_features(self) -> int:
        return self.geometry.padded_in_features

    @property
    def is_per_row(self) -> bool:
        return self.group_size == PER_ROW_GROUP_SIZE

    @property
    def device(self) -> torch.device:
        return self.packed.device

    @property
    def compute_dtype(self) -> torch.dtype:
        return self.scales.dtype

    @property
    def nbytes(self) -> int:
        """Bytes in memory including scales and offsets (the figure bandwidth is charged on)."""
        total = self.packed.numel() * 4 + self.scales.numel() * self.scales.element_size()
        if self.offsets is not None:
            total += self.offsets.numel() * self.offsets.element_size()
        return total

    def to(self, device: torch.device | str) -> QuantTensor:
        return replace(
            self,
            packed=self.packed.to(device),
            scales=self.scales.to(device),
            offsets=None if self.offsets is None else self.offsets.to(device),
        )

    def rows(self, start: int, stop: int) -> QuantTensor:
        """A view of rows ``[start, stop)`` (rows are independent under group-wise packing)."""
        return replace(
            self,
            packed=self.packed[start:stop],
            scales=self.scales[start:stop],
            offsets=None if self.offsets is None else self.offsets[start:stop],
            logical_shape=(stop - start, self.in_features),
            row_offset=self.row_offset + start,
        )

    def validate(self) -> None:
        g = self.geometry
        rows = self.packed.shape[0]
        if self.packed.dtype != torch.int32 or self.packed.ndim != 2:
            raise PackingError("packed must be a 2-D int32 tensor")
        if self.packed.shape[1] != g.words_per_row:
            raise PackingError(f"packed has {self.packed.shape[1]} words per row, geometry says {g.words_per_row}")
        if tuple(self.scales.shape) != (rows, g.num_groups):
            raise PackingError(f"scales shape {tuple(self.scales.shape)} != {(rows, g.num_groups)}")
        if self.offsets is not None and (
            self.offsets.shape != self.scales.shape or self.offsets.dtype != self.scales.dtype
        ):
            raise PackingError("offsets must match scales in shape and dtype")
        if self.layout != "linear":
            raise PackingError(f"unrecognised layout {self.layout!r}")

    @classmethod
    def from_codes(
        cls,
        codes: torch.Tensor,
        scales: torch.Tensor,
        offsets: torch.Tensor | None,
        *,
        bits: int,
        group_size: int = DEFAULT_GROUP_SIZE,
        in_features: int | None = None,
    ) -> QuantTensor:
        """Pack explicit codes ``[rows, padded_in_features]`` with given metadata."""
        in_features = int(codes.shape[-1] if in_features is None else in_features)
        g = row_geometry(bits, group_size, in_features)
        rows = codes.shape[0]
        if codes.shape[-1] != g.padded_in_features:
            raise PackingError(f"codes must cover the padded width {g.padded_in_features}")
        grouped = codes.reshape(rows, g.num_groups, g.effective_group)
        packed = pack_nbit(grouped, bits).reshape(rows, g.words_per_row)
        qt = cls(packed, scales, offsets, bits, g.group_size, in_features, (rows, in_features))
        qt.validate()
        return qt

    @classmethod
    def from_dense(
        cls,
        weight: torch.Tensor,
        *,
        bits: int,
        group_size: int = DEFAULT_GROUP_SIZE,
        symmetric: bool = False,
        compute_dtype: torch.dtype | None = None,
        row_offset: int = 0,
    ) -> QuantTensor:
        """Plain group-wise min/max quantization (``quant/tensor.py:239-396`` without clipping).

        Leading dims fold into rows, so a stacked expert weight ``[E, out, in]``
        becomes ``[E*out, in]`` and each expert keeps its own scales.  Scale and
        offset are rounded to the storage dtype *before* codes are derived
        (``docs/format-spec.md:198-204``); a constant group stores ``scale=0``,
        ``offset=value`` (``docs/format-spec.md:176-196``).
        """
        if weight.ndim < 2:
            raise PackingError(f"expected rank >= 2, got shape {tuple(weight.shape)}")
        logical_shape = tuple(weight.shape)
        in_features = logical_shape[-1]
        g = row_geometry(bits, group_size, in_features)
        compute_dtype = compute_dtype or (
            weight.dtype if weight.dtype in (torch.float16, torch.bfloat16) else torch.float16
        )
        rows2d = weight.reshape(-1, in_features).to(torch.float32)
        if g.padded_in_features != in_features:
            rows2d = torch.nn.functional.pad(rows2d, (0, g.padded_in_features - in_features))
        n = rows2d.shape[0]
        grouped = rows2d.reshape(n, g.num_groups, g.effective_group)
        qmax = (1 << bits) - 1
        lo = grouped.amin(-1)
        hi = grouped.amax(-1)
        constant = hi == lo
        if symmetric:
            half = 1 << (bits - 1)
            scale = torch.maximum(hi.abs(), lo.abs()) / max(half - 1, 1)
            scale = scale.to(compute_dtype)
            offset = (-half * scale.to(torch.float32)).to(compute_dtype)
        else:
            scale = ((hi - lo) / qmax).to(compute_dtype)
            offset = lo.to(compute_dtype)
        scale = torch.where(constant, torch.zeros_like(scale), scale)
        offset = torch.where(constant, lo.to(compute_dtype), offset)
        s32 = scale.to(torch.float32).unsqueeze(-1)
        o32 = offset.to(torch.float32).unsqueeze(-1)
        safe = torch.where(s32 == 0, torch.ones_like(s32), s32)
        codes = torch.round((grouped - o32) / safe).clamp_(0, qmax)
        codes = torch.where(s32 == 0, torch.zeros_like(codes), codes).to(torch.uint8)
        packed = pack_nbit(codes, bits).reshape(n, g.words_per_row)
        return cls(
            packed, scale, offset, bits, g.group_size, in_features, logical_shape,
            row_offset=row_offset, symmetric=symmetric,
        )

    def dequantize(self, *, dtype: torch.dtype | None = None) -> torch.Tensor:
        """Dense reconstruction, computed by the compiled dequant kernel."""
        from . import ops  # local import: ops depends on this module

        return ops.dequantize(self, dtype=dtype)
