"""Layer-side methods for serving frameworks: fused linear layers and the expert layer.

Mirrors the contract of the reference's serving plugins without importing a framework:

* ``ShardSpec`` / ``FusedPackedGeometry``: several shards of one fused layer (q/k/v,
  gate/up), each with its own bit width, stored back to back in flat 1-D ``qweight`` /
  ``scales`` / ``offsets`` buffers (reference ``integration/serving_common/geometry.py:338-367``,
  views ``:436-446``).
* ``DynQuantLinearMethod(quant_config, shards)`` with ``create_weights(layer,
  input_size_per_partition, output_partition_sizes, input_size, output_size, params_dtype,
  **extra)`` and ``apply(layer, x, bias=None)`` -- the signatures of
  ``integration/vllm_plugin/linear.py:84-186`` (SGLang's twin adds
  ``skip_block_quant_check``, accepted and ignored here).  ``apply`` makes ONE library call
  for all shards, bias folded into the store, instead of a GEMV per shard plus
  ``fused_shard_concat`` plus an add.
* ``DynQuantMoEMethod``: the fused-MoE method the reference refuses to provide
  (``integration/vllm_plugin/config.py:107-112``); hook shapes follow the host frameworks'
  fused-MoE method base (``create_weights(layer, num_experts, hidden_size,
  intermediate_size_per_partition, params_dtype, **extra)``, ``apply(layer, x, topk_weights,
  topk_ids)``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Sequence

import torch

from . import ops
from .format import QuantTensor, row_geometry


@dataclass(frozen=True)
class ShardSpec:
    """One shard of a fused layer: a row range with its own width."""

    name: str
    bits: int
    group_size: int
    out_features: int
    symmetric: bool = False


@dataclass(frozen=True)
class ShardPlan:
    spec: ShardSpec
    row_offset: int
    qweight_offset: int  # int32 elements into the flat qweight buffer
    qweight_numel: int
    scale_offset: int  # elements into the flat scales / offsets buffers
    scale_numel: int
    words_per_row: int
    num_groups: int


class FusedPackedGeometry:
    """Offsets of every shard inside the flat buffers of one fused layer."""

    def __init__(self, specs: Sequence[ShardSpec], in_features: int) -> None:
        if not specs:
            raise ValueError("a fused layer needs at least one shard")
        self.in_features = in_features
        plans: list[ShardPlan] = []
        row = qoff = soff = 0
        for spec in specs:
            g = row_geometry(spec.bits, spec.group_size, in_features)
            qn = spec.out_features * g.words_per_row
            sn = spec.out_features * g.num_groups
            plans.append(ShardPlan(spec, row, qoff, qn, soff, sn, g.words_per_row, g.num_groups))
            row += spec.out_features
            qoff += qn
            soff += sn
        self._plans = tuple(plans)
        self.out_features = row
        self.qweight_numel = qoff
        self.scale_numel = soff

    def __len__(self) -> int:
        return len(self._plans)

    def __getitem__(self, shard_id: int) -> ShardPlan:
        return self._plans[shard_id]

    def __iter__(self):
        return iter(self._plans)

    def plan_for_rows(self, dest_row: int, num_rows: int) -> ShardPlan:
        """The shard whose rows contain ``[dest_row, dest_row + num_rows)`` of the fused output --
        what a framework's weight loader names when it places (part of) one checkpoint module."""
        for plan in self._plans:
            if plan.row_offset <= dest_row and dest_row + num_rows <= plan.row_offset + plan.spec.out_features:
                return plan
        raise ValueError(
            f"rows [{dest_row}, {dest_row + num_rows}) do not lie inside one shard of "
            f"{[(p.spec.name, p.row_offset, p.spec.out_features) for p in self._plans]}"
        )

    def place(self, flat: torch.Tensor, kind: str, loaded: torch.Tensor, *, dest_row: int, num_rows: int,
              src_row: int, columns: slice | None = None) -> None:
        """Copy ``loaded[src_row : src_row + num_rows]`` (optionally a column slice of it: an input
        shard) into rows ``[dest_row, +num_rows)`` of the flat ``qweight`` or ``scales``/``offsets``
        buffer.  Pure placement: shapes must match exactly, nothing is repacked or converted
        (reference ``integration/vllm_plugin/parameter.py:158-183``)."""
        if kind not in ("qweight", "scale"):
            raise ValueError(f"unknown buffer kind {kind!r}")
        plan = self.plan_for_rows(dest_row, num_rows)
        per_row = plan.words_per_row if kind == "qweight" else plan.num_groups
        base = plan.qweight_offset if kind == "qweight" else plan.scale_offset
        start = base + (dest_row - plan.row_offset) * per_row
        dest = flat[start : start + num_rows * per_row].view(num_rows, per_row)
        source = loaded.narrow(0, src_row, num_rows)
        if columns is not None:
            source = source[:, columns]
        if source.shape != dest.shape:
            raise ValueError(
                f"{plan.spec.name}: the checkpoint tensor gives {tuple(source.shape)} for this rank but "
                f"{plan.spec.bits}-bit at group_size={plan.spec.group_size} needs {tuple(dest.shape)}; the "
                f"quantization map and the weights were written by different runs"
            )
        dest.copy_(source)

    def view_qweight(self, flat: torch.Tensor, shard_id: int) -> torch.Tensor:
        p = self._plans[shard_id]
        return flat[p.qweight_offset : p.qweight_offset + p.qweight_numel].view(p.spec.out_features, p.words_per_row)

    def view_scale(self, flat: torch.Tensor, shard_id: int) -> torch.Tensor:
        p = self._plans[shard_id]
        return flat[p.scale_offset : p.scale_offset + p.scale_numel].view(p.spec.out_features, p.num_groups)


@dataclass(frozen=True)
class InputSplit:
    """A packed row divided over ranks along its INPUT axis (the o_proj / down_proj placement)."""

    in_features: int  # per rank
    num_groups: int   # per rank
    words: int        # per rank

    def word_slice(self, rank: int) -> slice:
        return slice(rank * self.words, (rank + 1) * self.words)

    def group_slice(self, rank: int) -> slice:
        return slice(rank * self.num_groups, (rank + 1) * self.num_groups)


def input_axis_split(bits: int, group_size: int, in_features: int, world: int, name: str = "<layer>") -> InputSplit:
    """Words and groups each of ``world`` ranks owns of a row of ``in_features`` values.  Legal
    only on group boundaries -- a group's words, scale and offset move together -- and never for a
    per-row-grouped tensor (reference ``integration/serving_common/geometry.py:481-551``)."""
    full = row_geometry(bits, group_size, in_features)
    if world <= 0:
        raise ValueError(f"the number of ranks must be positive, got {world}")
    if world == 1:
        return InputSplit(in_features, full.num_groups, full.words_per_row)
    if full.is_per_row:
        raise ValueError(
            f"{name} has one group spanning its {in_features} inputs and cannot be split over {world} ranks: "
            f"every rank would need the one scale of a group it holds a part of"
        )
    if in_features % world:
        raise ValueError(f"{name}: in_features={in_features} is not divisible by {world} ranks")
    per = in_features // world
    if per % full.effective_group:
        raise ValueError(
            f"{name}: {world} ranks get {per} of {in_features} inputs each, which is not a whole number of groups "
            f"of {full.effective_group} values; use a rank count dividing {in_features // full.effective_group}"
        )
    part = row_geometry(bits, group_size, per)
    if part.words_per_row * world != full.words_per_row:
        raise ValueError(f"{name}: {world} slices of {part.words_per_row} words do not tile {full.words_per_row}")
    return InputSplit(per, part.num_groups, part.words_per_row)


def match_shards_to_partitions(shards: Sequence[ShardSpec], output_partition_sizes: Sequence[int]) -> list[ShardSpec]:
    """Check the quantization map describes this layer: one shard per output partition, sizes equal."""
    if len(shards) != len(output_partition_sizes):
        raise ValueError(
            f"the quantization map has {len(shards)} shards ({[s.name for s in shards]}) but the layer has "
            f"{len(output_partition_sizes)} output partitions"
        )
    for spec, size in zip(shards, output_partition_sizes):
        if spec.out_features != size:
            raise ValueError(f"shard {spec.name} has {spec.out_features} rows but its partition has {size}")
    return list(shards)


class DynQuantLinearMethod:
    """Quantization method of a (possibly fused) linear layer."""

    def __init__(self, quant_config: Any, shards: Sequence[ShardSpec]) -> None:
        self.quant_config = quant_config
        self.shards = list(shards)

    def create_weights(
        self,
        layer: torch.nn.Module,
        input_size_per_partition: int,
        output_partition_sizes: list[int],
        input_size: int,
        output_size: int,
        params_dtype: torch.dtype,
        **extra_weight_attrs: Any,
    ) -> None:
        del output_size
        specs = match_shards_to_partitions(self.shards, output_partition_sizes)
        split = None
        if input_size_per_partition != input_size:
            # row-parallel placement: this rank holds a slice of the input axis, legal only on
            # group boundaries (reference serving_common/geometry.py:481-551); the framework's
            # RowParallelLinear all-reduces the partial sums apply() returns
            if len(specs) != 1:
                raise ValueError(
                    f"the input-sharded layer {[s.name for s in specs]} has more than one fused shard: every "
                    f"width implies its own words per rank, so the word axis has no single split"
                )
            split = input_axis_split(specs[0].bits, specs[0].group_size, input_size,
                                     input_size // input_size_per_partition, specs[0].name)
        geometry = FusedPackedGeometry(specs, input_size_per_partition)
        device = extra_weight_attrs.get("device")
        layer.dynquant_geometry = geometry
        layer.dynquant_row_split = split
        layer.dynquant_in_features = input_size_per_partition
        for name, numel, dtype in (
            ("qweight", geometry.qweight_numel, torch.int32),
            ("scales", geometry.scale_numel, params_dtype),
            ("offsets", geometry.scale_numel, params_dtype),
        ):
            layer.register_parameter(
                name, torch.nn.Parameter(torch.empty(numel, dtype=dtype, device=device), requires_grad=False)
            )

    @staticmethod
    def load_shard(layer: torch.nn.Module, shard_id: int, weight: QuantTensor) -> None:
        """Copy one packed shard into its span of the flat buffers (what the framework's weight
        loader does through ``load_merged_column_weight`` / ``load_qkv_weight``)."""
        geometry: FusedPackedGeometry = layer.dynquant_geometry
        plan = geometry[shard_id]
        if (weight.bits, weight.num_rows, weight.in_features) != (plan.spec.bits, plan.spec.out_features, geometry.in_features):
            raise ValueError(f"shard {plan.spec.name}: tensor does not match its spec")
        geometry.view_qweight(layer.qweight.data, shard_id).copy_(weight.packed)
        geometry.view_scale(layer.scales.data, shard_id).copy_(weight.scales)
        if weight.offsets is None:
            geometry.view_scale(layer.offsets.data, shard_id).zero_()
        else:
            geometry.view_scale(layer.offsets.data, shard_id).copy_(weight.offsets)

    def shard_tensor(self, layer: torch.nn.Module, shard_id: int) -> QuantTensor:
        """A QuantTensor viewing one shard of the flat buffers (no copy)."""
        geometry: FusedPackedGeometry = layer.dynquant_geometry
        plan = geometry[shard_id]
        return QuantTensor(
            packed=geometry.view_qweight(layer.qweight.data, shard_id),
            scales=geometry.view_scale(layer.scales.data, shard_id),
            offsets=geometry.view_scale(layer.offsets.data, shard_id),
            bits=plan.spec.bits,
            group_size=plan.spec.group_size,
            in_features=geometry.in_features,
            logical_shape=(plan.spec.out_features, geometry.in_features),
            row_offset=plan.row_offset,
            symmetric=plan.spec.symmetric,
        )

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        geometry: FusedPackedGeometry = layer.dynquant_geometry
        shards = [self.shard_tensor(layer, i) for i in range(len(geometry))]
        lead = x.shape[:-1]
        flat = x.reshape(-1, geometry.in_features)
        if flat.shape[0] <= ops.gemv_max_rows():
            if bias is not None and bias.dtype != flat.dtype:
                bias = bias.to(flat.dtype)
            out = ops.gemv_shards(flat.contiguous(), shards, None if bias is None else bias.contiguous())
        elif flat.shape[0] <= ops.GEMV_CHUNKED_MAX_ROWS:
            if bias is not None and bias.dtype != flat.dtype:
                bias = bias.to(flat.dtype)
            out = ops.gemv_row_chunks(flat.contiguous(), shards, None if bias is None else bias.contiguous())
        else:
            parts = [
                torch.nn.functional.linear(flat, ops.dequant(*ops._kernel_args(qt)).to(flat.dtype)) for qt in shards
            ]
            out = parts[0] if len(parts) == 1 else torch.cat(parts, dim=-1)
            if bias is not None:
                out = out + bias
        return out.reshape(*lead, geometry.out_features)


class DynQuantMoEMethod:
    """Quantization method of a fused expert layer over packed banks."""

    def __init__(self, quant_config: Any, *, bits_gate_up: int, bits_down: int, group_size: int = 128) -> None:
        self.quant_config = quant_config
        self.bits_gate_up = bits_gate_up
        self.bits_down = bits_down
        self.group_size = group_size

    def create_weights(self, layer: torch.nn.Module, num_experts: int, hidden_size: int,
                       intermediate_size_per_partition: int, params_dtype: torch.dtype,
                       **extra_weight_attrs: Any) -> None:
        device = extra_weight_attrs.get("device")
        inter = intermediate_size_per_partition
        layer.dynquant_moe = (num_experts, hidden_size, inter)
        for prefix, rows, k, bits in (
            ("w13", num_experts * 2 * inter, hidden_size, self.bits_gate_up),
            ("w2", num_experts * hidden_size, inter, self.bits_down),
        ):
            g = row_geometry(bits, self.group_size, k)
            layer.register_parameter(f"{prefix}_qweight", torch.nn.Parameter(
                torch.empty(rows, g.words_per_row, dtype=torch.int32, device=device), requires_grad=False))
            for kind in ("scales", "offsets"):
                layer.register_parameter(f"{prefix}_{kind}", torch.nn.Parameter(
                    torch.empty(rows, g.num_groups, dtype=params_dtype, device=device), requires_grad=False))

    @staticmethod
    def load_banks(layer: torch.nn.Module, gate_up: QuantTensor, down: QuantTensor) -> None:
        for prefix, qt in (("w13", gate_up), ("w2", down)):
            getattr(layer, f"{prefix}_qweight").data.copy_(qt.packed)
            getattr(layer, f"{prefix}_scales").data.copy_(qt.scales)
            getattr(layer, f"{prefix}_offsets").data.copy_(qt.offsets)

    def _bank(self, layer: torch.nn.Module, prefix: str, bits: int, k: int) -> QuantTensor:
        packed = getattr(layer, f"{prefix}_qweight").data
        return QuantTensor(packed, getattr(layer, f"{prefix}_scales").data, getattr(layer, f"{prefix}_offsets").data,
                           bits, self.group_size, k, (packed.shape[0], k))

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, topk_weights: torch.Tensor,
              topk_ids: torch.Tensor, **_: Any) -> torch.Tensor:
        """``topk_weights`` are used as given (renormalise in the router if the model does)."""
        num_experts, hidden, inter = layer.dynquant_moe
        gate_up = self._bank(layer, "w13", self.bits_gate_up, hidden)
        down = self._bank(layer, "w2", self.bits_down, inter)
        lead = x.shape[:-1]
        flat = x.reshape(-1, hidden).contiguous()
        out = torch.empty_like(flat)
        limit = ops.moe_max_tokens()
        ids = topk_ids.reshape(flat.shape[0], -1).to(torch.int32)
        w = topk_weights.reshape(flat.shape[0], -1).to(torch.float32)
        for start in range(0, flat.shape[0], limit):  # decode batches fit one call; longer inputs chunk
            stop = min(start + limit, flat.shape[0])
            out[start:stop] = ops.moe_gemv(flat[start:stop].contiguous(), ids[start:stop].contiguous(),
                                           w[start:stop].contiguous(), gate_up, down, num_experts=num_experts)
        return out.reshape(*lead, hidden)
