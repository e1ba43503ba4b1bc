"""vLLM adapter: serve a packed checkpoint on the sm_100a kernels through vLLM's extension points.

    from dynquant_b200.vllm_plugin import register; register()

adds ``quant_method: "dynquant"`` to vLLM's quantization registry
(``register_quantization_config``), the same hook the reference's plugin uses
(``integration/vllm_plugin/__init__.py:49-74``).  This module imports vLLM and is therefore
never imported by the package itself.  What it provides, interface for interface:

* :class:`DynQuantConfig` (``QuantizationConfig``) -- ``integration/vllm_plugin/config.py:38-112``:
  parses ``config.json -> quantization_config`` (:class:`dynquant_b200.checkpoint.QuantizationConfig`)
  and hands every layer its own method.  Where the reference RAISES on a fused-MoE layer
  (``config.py:107-112``) this one returns :class:`DynQuantMoEMethod`.
* :class:`DynQuantPackedParameter` (``BasevLLMParameter``) -- ``parameter.py:41-183``: a flat
  buffer for a fused layer whose shards differ in width, with the four placement hooks of
  vLLM's v2 weight loader (column-parallel, merged-column, QKV with replicated KV heads,
  row-parallel on group boundaries).  Placement only: a load is a strided copy and a shape check.
* :class:`DynQuantLinearMethod` (``LinearMethodBase``) and :class:`DynQuantEmbeddingMethod` --
  ``linear.py:67-268``.  ``apply`` issues ONE launch for all shards of a fused layer with the
  bias folded into the store, instead of a launch per shard, an opaque concat and an add.
* :class:`DynQuantMoEMethod` (``FusedMoEMethodBase``) -- no reference counterpart: packed expert
  banks ``[E, rows, words]`` run by ``dq_moe_gemv``.

The placement arithmetic lives in :mod:`dynquant_b200.plugin` (importable with torch alone).
"""

from __future__ import annotations

from typing import Any, Callable, Mapping, Sequence

import torch
from vllm.model_executor.layers.fused_moe.fused_moe_method_base import FusedMoEMethodBase
from vllm.model_executor.layers.linear import (
    LinearBase,
    LinearMethodBase,
    UnquantizedLinearMethod,
    register_weight_loader_v2_supported_method,
)
from vllm.model_executor.layers.quantization.base_config import QuantizationConfig, QuantizeMethodBase
from vllm.model_executor.layers.vocab_parallel_embedding import ParallelLMHead, UnquantizedEmbeddingMethod
from vllm.model_executor.parameter import BasevLLMParameter
from vllm.model_executor.utils import set_weight_attrs

from . import ops
from . import plugin as core
from .checkpoint import QUANT_METHOD, ModuleSpec
from .checkpoint import QuantizationConfig as Schema
from .format import QuantTensor, row_geometry

MIN_CAPABILITY = 100  # sm_100a: the only architecture the library is compiled for
_MOE_PACKAGE = "vllm.model_executor.layers.fused_moe"


def register() -> None:
    """Add ``dynquant`` to vLLM's quantization registry.  Idempotent."""
    from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS, register_quantization_config

    if QUANT_METHOD not in QUANTIZATION_METHODS:
        register_quantization_config(QUANT_METHOD)(DynQuantConfig)


def expand_fused_prefix(prefix: str, packed_modules_mapping: Mapping[str, Sequence[str]]) -> list[str]:
    """``...self_attn.qkv_proj`` -> the checkpoint modules it was fused from; itself if unfused."""
    if not prefix:
        return [prefix]
    head, _, leaf = prefix.rpartition(".")
    parts = packed_modules_mapping.get(leaf)
    if not parts or list(parts) == [leaf]:
        return [prefix]
    return [f"{head}.{p}" if head else p for p in parts]


def is_fused_moe_class(cls: type) -> bool:
    """vLLM's expert layer, recognised by the package that defines any of its bases (the class
    itself has been renamed between vLLM releases)."""
    return any(b.__module__ == _MOE_PACKAGE or b.__module__.startswith(_MOE_PACKAGE + ".") for b in cls.__mro__)


class DynQuantConfig(QuantizationConfig):
    """Per-module bit widths: every layer is built with the width its checkpoint module has."""

    def __init__(self, schema: Schema) -> None:
        super().__init__()
        self.schema = schema

    def __repr__(self) -> str:
        widths = sorted({spec.bits for spec in self.schema.modules.values()})
        return f"DynQuantConfig(modules={len(self.schema.modules)}, bits={widths}, group_size={self.schema.group_size})"

    def get_name(self) -> str:
        return QUANT_METHOD

    def get_supported_act_dtypes(self) -> list[torch.dtype]:
        return [torch.half, torch.bfloat16]

    @classmethod
    def get_min_capability(cls) -> int:
        return MIN_CAPABILITY

    @staticmethod
    def get_config_filenames() -> list[str]:
        return []  # everything is in config.json

    @classmethod
    def from_config(cls, config: dict[str, Any]) -> "DynQuantConfig":
        return cls(Schema.from_dict(config))

    def resolve_shards(self, prefix: str) -> list[tuple[str, ModuleSpec]] | None:
        """Checkpoint modules behind one serving layer; ``None`` if none of them is packed.  A
        fused layer with some shards packed and others dense is refused: its shards share one
        buffer (reference ``serving_common/schema.py:284-328``)."""
        names = expand_fused_prefix(prefix, getattr(self, "packed_modules_mapping", {}) or {})
        found = [(name, self.schema.get(name)) for name in names]
        present = [(name, spec) for name, spec in found if spec is not None]
        if not present:
            return None
        if len(present) != len(found):
            missing = [name for name, spec in found if spec is None]
            raise ValueError(
                f"{prefix} fuses {names}, but {missing} are not in the quantization map while the others are; "
                f"the shards of a fused layer share one packed buffer, so all or none must be packed"
            )
        return present

    def get_quant_method(self, layer: torch.nn.Module, prefix: str) -> QuantizeMethodBase | None:
        if is_fused_moe_class(type(layer)):
            banks = self.resolve_expert_banks(prefix)
            return None if banks is None else DynQuantMoEMethod(layer.moe_config, self, *banks)
        if isinstance(layer, ParallelLMHead):
            shards = self.resolve_shards(prefix) if self.schema.lm_head_quantized else None
            return UnquantizedEmbeddingMethod() if shards is None else DynQuantEmbeddingMethod(self, shards)
        if isinstance(layer, LinearBase):
            shards = self.resolve_shards(prefix)
            return UnquantizedLinearMethod() if shards is None else DynQuantLinearMethod(self, shards)
        return None  # embeddings, norms: the exporter left them dense

    def resolve_expert_banks(self, prefix: str) -> tuple[ModuleSpec, ModuleSpec] | None:
        """Widths of the two banks of an expert layer: modules ``<prefix>.gate_up_proj`` and
        ``<prefix>.down_proj`` of the map (stacked banks folded to rows, reference
        ``graph/experts.py:35-43``, ``quant/tensor.py:253-255``)."""
        gate_up, down = self.schema.get(f"{prefix}.gate_up_proj"), self.schema.get(f"{prefix}.down_proj")
        if gate_up is None and down is None:
            return None
        if gate_up is None or down is None:
            raise ValueError(f"{prefix}: one expert bank is packed and the other is not")
        return gate_up, down


# ---------------------------------------------------------------------------------------------
# linear layers
# ---------------------------------------------------------------------------------------------


class DynQuantPackedParameter(BasevLLMParameter):
    """Flat ``qweight`` / ``scales`` / ``offsets`` buffer of one (possibly fused) linear layer.

    ``output_dim`` / ``input_dim`` describe the LOADED 2-D tensor (vLLM slices that); no
    ``packed_dim`` is declared because packing runs along the input axis, not the output one.
    """

    def __new__(cls, data: torch.Tensor, **kwargs: Any):
        return super().__new__(cls, data=data, **kwargs)

    def __init__(self, *, data: torch.Tensor, weight_loader: Callable[..., None] | None,
                 geometry: core.FusedPackedGeometry, kind: str, row_split: core.InputSplit | None = None) -> None:
        super().__init__(data=data, weight_loader=weight_loader)
        self._geometry, self._kind, self._row_split = geometry, kind, row_split

    output_dim = property(lambda self: 0)
    input_dim = property(lambda self: 1)
    geometry = property(lambda self: self._geometry)

    def _columns(self) -> slice | None:
        if self._row_split is None:
            return None
        return self._row_split.word_slice(self.tp_rank) if self._kind == "qweight" else self._row_split.group_slice(self.tp_rank)

    def _place(self, loaded: torch.Tensor, dest_row: int, num_rows: int, src_row: int) -> None:
        self._geometry.place(self.data, self._kind, loaded, dest_row=dest_row, num_rows=num_rows, src_row=src_row,
                             columns=self._columns())

    def load_column_parallel_weight(self, loaded_weight: torch.Tensor) -> None:
        rows = self._geometry.out_features
        self._place(loaded_weight, 0, rows, self.tp_rank * rows)

    def load_merged_column_weight(self, loaded_weight: torch.Tensor, **kwargs: Any) -> None:
        # shard_offset / shard_size are this rank's rows of the fused output; the loaded tensor spans all ranks
        size = int(kwargs["shard_size"])
        self._place(loaded_weight, int(kwargs["shard_offset"]), size, self.tp_rank * size)

    def load_qkv_weight(self, loaded_weight: torch.Tensor, **kwargs: Any) -> None:
        # fewer KV heads than ranks: `num_heads` ranks read the SAME k / v rows
        size = int(kwargs["shard_size"])
        replicas = int(kwargs.get("num_heads", 1)) or 1
        index = self.tp_rank if kwargs["shard_id"] == "q" else self.tp_rank // replicas
        self._place(loaded_weight, int(kwargs["shard_offset"]), size, index * size)

    def load_row_parallel_weight(self, loaded_weight: torch.Tensor) -> None:
        self._place(loaded_weight, 0, self._geometry.out_features, 0)


def _shard_specs(shards: Sequence[tuple[str, ModuleSpec]], sizes: Sequence[int]) -> list[core.ShardSpec]:
    if len(shards) != len(sizes):
        raise ValueError(f"{len(shards)} checkpoint modules {[n for n, _ in shards]} for {len(sizes)} output partitions")
    return [core.ShardSpec(name, spec.bits, spec.group_size, int(size), spec.symmetric)
            for (name, spec), size in zip(shards, sizes)]


@register_weight_loader_v2_supported_method
class DynQuantLinearMethod(LinearMethodBase):
    """A linear layer whose fused shards may each have their own width.  The decorator puts the
    class on vLLM's v2-loader list: only the v2 loader calls the parameter's placement hooks."""

    def __init__(self, quant_config: DynQuantConfig | None, shards: Sequence[tuple[str, ModuleSpec]]) -> None:
        self.quant_config = quant_config
        self.shards = list(shards)

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: list[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs: Any) -> None:
        specs = _shard_specs(self.shards, output_partition_sizes)
        inner = core.DynQuantLinearMethod(self.quant_config, specs)
        loader = extra_weight_attrs.get("weight_loader")
        rest = {k: v for k, v in extra_weight_attrs.items() if k != "weight_loader"}  # set_weight_attrs refuses to overwrite
        inner.create_weights(layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                             params_dtype, device=rest.pop("device", None))
        layer.dynquant_method = inner
        for name, kind in (("qweight", "qweight"), ("scales", "scale"), ("offsets", "scale")):
            plain = getattr(layer, name)
            delattr(layer, name)
            param = DynQuantPackedParameter(data=plain.data, weight_loader=loader, geometry=layer.dynquant_geometry,
                                            kind=kind, row_split=layer.dynquant_row_split)
            layer.register_parameter(name, param)
            set_weight_attrs(param, rest)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        return layer.dynquant_method.apply(layer, x, bias)


class DynQuantEmbeddingMethod(DynQuantLinearMethod):
    """Packed vocabulary table (``embed_tokens``, a quantized or tied lm_head): 2-D parameters,
    because ``VocabParallelEmbedding.weight_loader`` copies and zero-fills along dim 0."""

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: list[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs: Any) -> None:
        if len(self.shards) != 1:
            raise ValueError(f"an embedding table cannot be fused, got {[n for n, _ in self.shards]}")
        _, spec = self.shards[0]
        rows = sum(output_partition_sizes)
        g = row_geometry(spec.bits, spec.group_size, input_size_per_partition)
        layer.dynquant_spec, layer.dynquant_in_features = spec, input_size_per_partition
        for name, cols, dtype in (("qweight", g.words_per_row, torch.int32), ("scales", g.num_groups, params_dtype),
                                  ("offsets", g.num_groups, params_dtype)):
            # zeros: a padded vocabulary row must decode to the zero vector (code 0, scale 0, offset 0)
            param = torch.nn.Parameter(torch.zeros(rows, cols, dtype=dtype), requires_grad=False)
            layer.register_parameter(name, param)
            set_weight_attrs(param, {"output_dim": 0, "input_dim": 1})
            set_weight_attrs(param, extra_weight_attrs)

    @staticmethod
    def _table(layer: torch.nn.Module) -> QuantTensor:
        spec, k = layer.dynquant_spec, layer.dynquant_in_features
        return QuantTensor(layer.qweight.data, layer.scales.data, layer.offsets.data, spec.bits, spec.group_size, k,
                           (layer.qweight.shape[0], k), symmetric=spec.symmetric)

    def embedding(self, layer: torch.nn.Module, input_: torch.Tensor) -> torch.Tensor:
        return ops.embedding_lookup(self._table(layer), input_)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        return ops.quantized_matmul(x, self._table(layer), bias)

    def tie_weights(self, layer: torch.nn.Module, embed_tokens: torch.nn.Module) -> torch.nn.Module:
        for name in ("qweight", "scales", "offsets"):  # all three buffers, not just a `weight`
            setattr(layer, name, getattr(embed_tokens, name))
        layer.dynquant_spec, layer.dynquant_in_features = embed_tokens.dynquant_spec, embed_tokens.dynquant_in_features
        return layer


# ---------------------------------------------------------------------------------------------
# expert layers
# ---------------------------------------------------------------------------------------------


def _bank_loader(param: torch.nn.Parameter, loaded_weight: torch.Tensor, weight_name: str | None = None,
                 shard_id: str | None = None, expert_id: int | None = None, **_: Any) -> None:
    """Weight loader of a packed bank ``[E, rows, cols]``.  A whole bank (``expert_id`` None) arrives
    folded to rows ``[E * rows, cols]``; a per-expert tensor names its half of ``w13`` through
    ``shard_id``: ``w1`` = gate rows, ``w3`` = up rows (gate before up, reference
    ``graph/experts.py:35-43``), ``w2`` = the down bank."""
    data = param.data
    if expert_id is None:
        if loaded_weight.numel() != data.numel():
            raise ValueError(f"{weight_name}: bank of {tuple(loaded_weight.shape)} for a buffer of {tuple(data.shape)}")
        data.view(-1, data.shape[-1]).copy_(loaded_weight.reshape(-1, data.shape[-1]))
        return
    rows = data.shape[1]
    if shard_id in ("w1", "w3"):
        half = rows // 2
        dest = data[expert_id, :half] if shard_id == "w1" else data[expert_id, half:]
    else:
        dest = data[expert_id]
    if dest.shape != loaded_weight.shape:
        raise ValueError(f"{weight_name}: expert {expert_id} {shard_id} gives {tuple(loaded_weight.shape)}, "
                         f"the buffer needs {tuple(dest.shape)}")
    dest.copy_(loaded_weight)


class DynQuantMoEMethod(FusedMoEMethodBase):
    """Packed expert banks on ``dq_moe_gemv``: gate/up and down GEMVs grouped per expert, SwiGLU
    between them, the weighted combine in slot order.  ``topk_weights`` are used as given."""

    def __init__(self, moe: Any, quant_config: DynQuantConfig | None, gate_up: ModuleSpec, down: ModuleSpec) -> None:
        super().__init__(moe)
        if gate_up.group_size != down.group_size:
            raise ValueError("the two banks of an expert layer must share one group size")
        self.quant_config = quant_config
        self.inner = core.DynQuantMoEMethod(quant_config, bits_gate_up=gate_up.bits, bits_down=down.bits,
                                            group_size=gate_up.group_size)

    def create_weights(self, layer: torch.nn.Module, num_experts: int, hidden_size: int,
                       intermediate_size_per_partition: int, params_dtype: torch.dtype, **extra_weight_attrs: Any) -> None:
        rest = {k: v for k, v in extra_weight_attrs.items() if k != "weight_loader"}
        self.inner.create_weights(layer, num_experts, hidden_size, intermediate_size_per_partition, params_dtype,
                                  device=rest.pop("device", None))
        for prefix, rows in (("w13", 2 * intermediate_size_per_partition), ("w2", hidden_size)):
            for kind in ("qweight", "scales", "offsets"):
                flat = getattr(layer, f"{prefix}_{kind}")
                delattr(layer, f"{prefix}_{kind}")
                param = torch.nn.Parameter(flat.data.view(num_experts, rows, flat.shape[-1]), requires_grad=False)
                layer.register_parameter(f"{prefix}_{kind}", param)
                set_weight_attrs(param, {"weight_loader": _bank_loader, **rest})

    def get_fused_moe_quant_config(self, layer: torch.nn.Module):
        return None  # no modular-kernel quantization: the packed kernel is the whole expert computation

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
              shared_experts: Any = None, shared_experts_input: torch.Tensor | None = None) -> torch.Tensor:
        if shared_experts is not None:
            from vllm.model_executor.layers.fused_moe.runner.shared_experts import SharedExpertsOrder

            shared_experts.apply(shared_experts_input, SharedExpertsOrder.MK_INTERNAL_OVERLAPPED)
        return self.inner.apply(_Folded(layer), x, topk_weights, topk_ids)


class _Folded:
    """A layer's banks seen folded to rows ``[E * rows, cols]`` -- the layout ``dq_moe_gemv`` takes."""

    def __init__(self, layer: torch.nn.Module) -> None:
        self._layer = layer
        self.dynquant_moe = layer.dynquant_moe

    def __getattr__(self, name: str):
        value = getattr(self._layer, name)
        if isinstance(value, torch.Tensor) and value.dim() == 3:
            return torch.nn.Parameter(value.data.view(-1, value.shape[-1]), requires_grad=False)
        return value
