"""Packed checkpoints: read and write the directory the reference's exporter produces.

Layout (reference ``quant/checkpoint.py:20-29, 331-369``, ``docs/format-spec.md`` section 6):
HF-style ``model.safetensors`` -- or ``model-0000i-of-0000N.safetensors`` shards plus
``model.safetensors.index.json`` -- where every quantized module ``<name>`` contributes

    <name>.qweight  int32      [rows, groups * words_per_group]
    <name>.scales   fp16/bf16  [rows, groups]
    <name>.offsets  fp16/bf16  [rows, groups]   (optional)

a row-partitioned module stores shard ``i`` under ``<name>.s<i>`` (``constants.py:134``), and
every other tensor (norms, embeddings, biases) keeps its own key.  The widths live in
``config.json -> quantization_config`` (``integration/serving_common/schema.py:152-245``):
``quant_method: "dynquant"``, ``checkpoint_format: "dynquant-packed"``, ``schema_version``,
file-level ``group_size`` / ``symmetric`` defaults and ``modules: {name: {bits, [group_size],
[symmetric], [out_features]}}`` (a bare integer is accepted for ``{bits}``).

``load_packed_checkpoint`` turns such a directory into :class:`~dynquant_b200.format.QuantTensor`
objects ready for the kernels -- the tensors are used as stored, nothing is repacked --, and
``save_packed_checkpoint`` writes one the reference's loaders accept.  Nothing here quantizes:
encoding is :meth:`QuantTensor.from_dense`.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping

import torch

from .format import BIT_OPTIONS as SUPPORTED_BITS
from .format import PER_ROW_GROUP_SIZE, QuantTensor, row_geometry

QUANT_METHOD = "dynquant"
CHECKPOINT_FORMAT = "dynquant-packed"
SCHEMA_VERSION = 1
CONFIG_FILENAME = "config.json"
WEIGHTS_FILENAME = "model.safetensors"
WEIGHTS_INDEX_FILENAME = "model.safetensors.index.json"
SHARD_PATTERN = "model-{index:05d}-of-{total:05d}.safetensors"
DEFAULT_GROUP_SIZE = 128
DEFAULT_SHARD_BYTES = 4 * 1024**3
SUFFIXES = ("qweight", "scales", "offsets")
_ROW_SHARD = re.compile(r"^(?P<name>.+)\.s(?P<index>\d+)$")


class CheckpointError(RuntimeError):
    """The directory is not a packed checkpoint this build can read."""


@dataclass(frozen=True)
class ModuleSpec:
    """Width of one checkpoint module (reference ``ModuleQuantSpec``)."""

    bits: int
    group_size: int = DEFAULT_GROUP_SIZE
    symmetric: bool = False
    out_features: int | None = None

    def __post_init__(self) -> None:
        if self.bits not in SUPPORTED_BITS:
            raise CheckpointError(
                f"bits={self.bits} is not one of {list(SUPPORTED_BITS)}; this checkpoint was written by a "
                f"different version of DynQuant"
            )
        if self.out_features is not None and self.out_features <= 0:
            raise CheckpointError(f"out_features must be positive, got {self.out_features}")


@dataclass(frozen=True)
class QuantizationConfig:
    """``config.json -> quantization_config`` (reference ``QuantizationConfigSchema``)."""

    modules: Mapping[str, ModuleSpec]
    group_size: int = DEFAULT_GROUP_SIZE
    symmetric: bool = False
    lm_head_quantized: bool = False
    modules_to_not_convert: tuple[str, ...] = ()
    version: str = ""

    @classmethod
    def from_dict(cls, config: Mapping[str, Any]) -> QuantizationConfig:
        method = config.get("quant_method")
        if method is not None and method != QUANT_METHOD:
            raise CheckpointError(f"quantization_config.quant_method is {method!r}, not {QUANT_METHOD!r}")
        schema_version = int(config.get("schema_version", SCHEMA_VERSION))
        if schema_version > SCHEMA_VERSION:
            raise CheckpointError(
                f"quantization_config block is schema v{schema_version}; this build reads up to v{SCHEMA_VERSION}"
            )
        fmt = config.get("checkpoint_format", CHECKPOINT_FORMAT)
        if fmt != CHECKPOINT_FORMAT:
            raise CheckpointError(
                f"checkpoint_format is {fmt!r}, not {CHECKPOINT_FORMAT!r}. Only a packed DynQuant checkpoint "
                f"holds tensors these kernels can read."
            )
        group_size = int(config.get("group_size", DEFAULT_GROUP_SIZE))
        symmetric = bool(config.get("symmetric", False))
        raw = config.get("modules")
        if not isinstance(raw, Mapping) or not raw:
            raise CheckpointError(
                "quantization_config.modules is missing or empty. DynQuant allocates a width per module, so the "
                "map is the configuration -- there is no single bit width to fall back on."
            )
        modules = {name: _spec_from_entry(name, entry, group_size, symmetric) for name, entry in raw.items()}
        return cls(
            modules=modules, group_size=group_size, symmetric=symmetric,
            lm_head_quantized=bool(config.get("lm_head_quantized", False)),
            modules_to_not_convert=tuple(config.get("modules_to_not_convert", ())),
            version=str(config.get("version", "")),
        )

    def to_dict(self) -> dict[str, Any]:
        def entry(spec: ModuleSpec) -> dict[str, Any]:
            out: dict[str, Any] = {"bits": spec.bits}  # only what differs from the file-level defaults
            if spec.group_size != self.group_size:
                out["group_size"] = spec.group_size
            if spec.symmetric != self.symmetric:
                out["symmetric"] = spec.symmetric
            if spec.out_features is not None:
                out["out_features"] = spec.out_features
            return out

        return {
            "quant_method": QUANT_METHOD,
            "checkpoint_format": CHECKPOINT_FORMAT,
            "schema_version": SCHEMA_VERSION,
            "version": self.version,
            "group_size": self.group_size,
            "symmetric": self.symmetric,
            "lm_head_quantized": self.lm_head_quantized,
            "modules_to_not_convert": list(self.modules_to_not_convert),
            "modules": {name: entry(spec) for name, spec in sorted(self.modules.items())},
        }

    def get(self, name: str) -> ModuleSpec | None:
        """The spec of a checkpoint module, or ``None`` if it stayed dense."""
        if name in self.modules_to_not_convert:
            return None
        return self.modules.get(name)


def _spec_from_entry(name: str, entry: Any, group_size: int, symmetric: bool) -> ModuleSpec:
    if isinstance(entry, int) and not isinstance(entry, bool):
        return ModuleSpec(entry, group_size, symmetric)
    if not isinstance(entry, Mapping):
        raise CheckpointError(
            f"quantization_config.modules[{name!r}] should be an int or an object with a 'bits' key, "
            f"got {type(entry).__name__}"
        )
    if "bits" not in entry:
        raise CheckpointError(f"quantization_config.modules[{name!r}] has no 'bits'")
    out_features = entry.get("out_features")
    return ModuleSpec(
        bits=int(entry["bits"]), group_size=int(entry.get("group_size", group_size)),
        symmetric=bool(entry.get("symmetric", symmetric)),
        out_features=None if out_features is None else int(out_features),
    )


@dataclass
class PackedCheckpoint:
    """A loaded packed checkpoint.

    ``modules[name]`` is the list of row shards of a module in ascending row order (one entry
    for almost every module); ``dense`` holds every other tensor under its own key; ``config``
    is the rest of ``config.json``.
    """

    quantization: QuantizationConfig
    modules: dict[str, list[QuantTensor]]
    dense: dict[str, torch.Tensor]
    config: dict[str, Any] = field(default_factory=dict)

    def tensor(self, name: str) -> QuantTensor:
        """The packed tensor of a module stored as one shard."""
        shards = self.modules[name]
        if len(shards) != 1:
            raise CheckpointError(f"{name} is stored as {len(shards)} row shards; use .modules[{name!r}]")
        return shards[0]

    @property
    def packed_bytes(self) -> int:
        return sum(qt.nbytes for shards in self.modules.values() for qt in shards)

    def linear(self, name: str):
        """A :class:`~dynquant_b200.runtime.DynQuantLinear` over a module's packed tensor, with
        the module's own ``<name>.bias`` when the checkpoint holds one."""
        from .runtime import DynQuantLinear

        return DynQuantLinear(self.tensor(name), self.dense.get(f"{name}.bias"))

    def fused(self, names: list[str]) -> list[QuantTensor]:
        """The shards of a server-side fused layer (``qkv_proj`` = q, k, v), in order: what
        :func:`dynquant_b200.ops.gemv_shards` and ``DynQuantLinearMethod.load_shard`` take."""
        out: list[QuantTensor] = []
        for name in names:
            out.extend(self.modules[name])
        return out


def _weight_files(path: Path) -> list[Path]:
    index = path / WEIGHTS_INDEX_FILENAME
    if index.exists():
        weight_map = json.loads(index.read_text(encoding="utf-8")).get("weight_map", {})
        names = sorted(set(weight_map.values()))
        missing = [n for n in names if not (path / n).exists()]
        if missing:
            raise CheckpointError(f"{index.name} names {missing}, which are not in {path}")
        return [path / n for n in names]
    files = sorted(path.glob("*.safetensors"))
    if not files:
        raise CheckpointError(f"no .safetensors file in {path}")
    return files


def _build_tensor(name: str, spec: ModuleSpec, parts: Mapping[str, torch.Tensor], in_features: int | None,
                  row_offset: int) -> QuantTensor:
    if "qweight" not in parts or "scales" not in parts:
        raise CheckpointError(f"{name}: the checkpoint holds {sorted(parts)} but a packed module needs qweight and scales")
    packed, scales, offsets = parts["qweight"], parts["scales"], parts.get("offsets")
    if packed.dtype != torch.int32 or packed.dim() != 2:
        raise CheckpointError(f"{name}.qweight must be a 2-D int32 tensor, got {packed.dtype} {tuple(packed.shape)}")
    if scales.dtype not in (torch.float16, torch.bfloat16) or scales.dim() != 2 or scales.shape[0] != packed.shape[0]:
        raise CheckpointError(f"{name}.scales must be fp16/bf16 [rows, groups], got {scales.dtype} {tuple(scales.shape)}")
    if offsets is not None and (offsets.shape != scales.shape or offsets.dtype != scales.dtype):
        raise CheckpointError(f"{name}.offsets must match scales, got {offsets.dtype} {tuple(offsets.shape)}")
    rows, words = int(packed.shape[0]), int(packed.shape[1])
    groups = int(scales.shape[1])
    if spec.group_size == PER_ROW_GROUP_SIZE:
        if groups != 1:
            raise CheckpointError(f"{name}: a per-row tensor has one group per row, the checkpoint has {groups}")
        # a per-row tensor's length is not implied by its shapes to better than a word
        k = in_features if in_features is not None else words * 32 // spec.bits
    else:
        k = in_features if in_features is not None else groups * spec.group_size
    geometry = row_geometry(spec.bits, spec.group_size, k)
    if geometry.num_groups != groups or geometry.words_per_row != words:
        raise CheckpointError(
            f"{name}: {spec.bits}-bit, group {spec.group_size}, in_features {k} implies {geometry.num_groups} groups "
            f"of {geometry.words_per_group} words, but the checkpoint stores scales {tuple(scales.shape)} and "
            f"qweight {tuple(packed.shape)}"
        )
    return QuantTensor(packed, scales, offsets, spec.bits, spec.group_size, k, (rows, k), row_offset=row_offset,
                       symmetric=spec.symmetric)


def load_packed_checkpoint(path: str | Path, *, device: str | torch.device = "cpu",
                           in_features: Mapping[str, int] | None = None) -> PackedCheckpoint:
    """Read a packed checkpoint directory.

    The input width of a module is taken, in this order, from ``in_features`` (an explicit
    per-module override), from the exporter's ``dynquant_manifest.json`` when the directory has
    one (``layers[name].in_features``; the reference writes it beside the weights,
    ``quant/checkpoint.py:109-200``), and otherwise from the stored shapes
    (``groups * group_size``) -- which over-states it for a module whose rows end in a
    zero-padded partial group.  Tensors are moved to ``device`` as stored.
    """
    from safetensors import safe_open

    path = Path(path)
    config_path = path / CONFIG_FILENAME
    if not config_path.exists():
        raise CheckpointError(f"{config_path} does not exist")
    config = json.loads(config_path.read_text(encoding="utf-8"))
    block = config.pop("quantization_config", None)
    if not isinstance(block, Mapping):
        raise CheckpointError(f"{config_path} has no quantization_config block: not a packed DynQuant checkpoint")
    quantization = QuantizationConfig.from_dict(block)

    tensors: dict[str, torch.Tensor] = {}
    for file in _weight_files(path):
        with safe_open(str(file), framework="pt", device="cpu") as handle:
            for key in handle.keys():
                if key in tensors:
                    raise CheckpointError(f"{key} appears in more than one weight file")
                tensors[key] = handle.get_tensor(key)

    # group <prefix>.<suffix> keys by prefix; a prefix is a module name or <module>.s<i>
    grouped: dict[str, dict[str, torch.Tensor]] = {}
    dense: dict[str, torch.Tensor] = {}
    for key, value in tensors.items():
        prefix, _, suffix = key.rpartition(".")
        base = _ROW_SHARD.match(prefix)
        module = base.group("name") if base else prefix
        if suffix in SUFFIXES and quantization.get(module) is not None:
            grouped.setdefault(prefix, {})[suffix] = value
        else:
            dense[key] = value.to(device)

    widths = _manifest_widths(path)
    widths.update(in_features or {})
    modules: dict[str, list[QuantTensor]] = {}
    for name, spec in quantization.modules.items():
        if name in quantization.modules_to_not_convert:
            continue
        if name in grouped:
            prefixes = [name]
        else:
            found = sorted(
                (int(m.group("index")), p) for p in grouped if (m := _ROW_SHARD.match(p)) and m.group("name") == name
            )
            if [i for i, _ in found] != list(range(len(found))) or not found:
                raise CheckpointError(
                    f"{name} is in the quantization map but the weight files hold no {name}.qweight "
                    f"(nor a complete run of {name}.s<i> shards)"
                )
            prefixes = [p for _, p in found]
        shards, row = [], 0
        for prefix in prefixes:
            qt = _build_tensor(prefix, spec, grouped[prefix], widths.get(name), row)
            shards.append(qt.to(device))
            row += qt.num_rows
        if spec.out_features is not None and row != spec.out_features:
            raise CheckpointError(f"{name}: the map says {spec.out_features} rows, the tensors hold {row}")
        modules[name] = shards
    return PackedCheckpoint(quantization, modules, dense, config)


MANIFEST_FILENAME = "dynquant_manifest.json"


def _manifest_widths(path: Path) -> dict[str, int]:
    """``in_features`` per module from the exporter's manifest, if the directory has one."""
    manifest = path / MANIFEST_FILENAME
    if not manifest.exists():
        return {}
    try:
        layers = json.loads(manifest.read_text(encoding="utf-8")).get("layers", {})
    except ValueError as exc:
        raise CheckpointError(f"{manifest} is not valid JSON: {exc}") from exc
    out = {}
    for name, entry in layers.items():
        if isinstance(entry, Mapping) and "in_features" in entry:
            out[name] = int(entry["in_features"])
    return out


def save_packed_checkpoint(
    output_dir: str | Path,
    modules: Mapping[str, QuantTensor | list[QuantTensor]],
    dense: Mapping[str, torch.Tensor] | None = None,
    *,
    config: Mapping[str, Any] | None = None,
    group_size: int = DEFAULT_GROUP_SIZE,
    symmetric: bool = False,
    modules_to_not_convert: tuple[str, ...] = (),
    version: str = "",
    max_shard_bytes: int = DEFAULT_SHARD_BYTES,
) -> tuple[str, ...]:
    """Write a packed checkpoint directory; returns the files written.

    ``modules`` maps a module name to its packed tensor (or its row shards, written as
    ``<name>.s<i>``); ``dense`` tensors are written under their own keys; ``config`` is the
    model's own ``config.json`` content, to which the ``quantization_config`` block is added.
    One ``model.safetensors`` and no index when everything fits ``max_shard_bytes``.
    """
    from safetensors.torch import save_file

    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    tensors: dict[str, torch.Tensor] = {}
    specs: dict[str, ModuleSpec] = {}
    for name, value in modules.items():
        shards = value if isinstance(value, list) else [value]
        if not shards:
            raise CheckpointError(f"{name}: no tensor to write")
        first = shards[0]
        for i, qt in enumerate(shards):
            if (qt.bits, qt.group_size, qt.in_features) != (first.bits, first.group_size, first.in_features):
                raise CheckpointError(f"{name}: row shards of one module share width, group size and in_features")
            prefix = name if len(shards) == 1 else f"{name}.s{i}"
            tensors[f"{prefix}.qweight"] = qt.packed
            tensors[f"{prefix}.scales"] = qt.scales
            if qt.offsets is not None:
                tensors[f"{prefix}.offsets"] = qt.offsets
        specs[name] = ModuleSpec(first.bits, first.group_size, first.symmetric, sum(qt.num_rows for qt in shards))
    for key, value in (dense or {}).items():
        if key in tensors:
            raise CheckpointError(f"{key} is both a dense tensor and part of a packed module")
        tensors[key] = value

    groups: list[dict[str, torch.Tensor]] = [{}]
    sizes = [0]
    for key in sorted(tensors):
        value = tensors[key].detach().cpu().contiguous()
        nbytes = value.numel() * value.element_size()
        if sizes[-1] and sizes[-1] + nbytes > max_shard_bytes:
            groups.append({})
            sizes.append(0)
        groups[-1][key] = value
        sizes[-1] += nbytes
    if len(groups) == 1:
        save_file(groups[0], str(out / WEIGHTS_FILENAME), metadata={"format": "pt"})
        files: tuple[str, ...] = (WEIGHTS_FILENAME,)
    else:
        names = [SHARD_PATTERN.format(index=i + 1, total=len(groups)) for i in range(len(groups))]
        weight_map: dict[str, str] = {}
        for file_name, group in zip(names, groups):
            save_file(group, str(out / file_name), metadata={"format": "pt"})
            weight_map.update(dict.fromkeys(group, file_name))
        index = {"metadata": {"total_size": sum(sizes)}, "weight_map": {k: weight_map[k] for k in sorted(weight_map)}}
        (out / WEIGHTS_INDEX_FILENAME).write_text(json.dumps(index, indent=2), encoding="utf-8")
        files = (*names, WEIGHTS_INDEX_FILENAME)

    quantization = QuantizationConfig(
        modules=specs, group_size=group_size, symmetric=symmetric,
        lm_head_quantized=any(name.split(".")[-1] == "lm_head" for name in specs),
        modules_to_not_convert=tuple(modules_to_not_convert), version=version,
    )
    payload = dict(config or {})
    payload["quantization_config"] = quantization.to_dict()
    (out / CONFIG_FILENAME).write_text(json.dumps(payload, indent=2, sort_keys=True), encoding="utf-8")
    return (*files, CONFIG_FILENAME)
