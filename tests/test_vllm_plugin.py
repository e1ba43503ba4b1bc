"""The vLLM adapter without a GPU: registration, per-layer dispatch, and tensor-parallel placement.

Placement is what tensor parallelism can break: which rows of a fused column-parallel layer and
which packed words of an input-sharded one each rank copies out of a checkpoint tensor spanning
all ranks.  As in the reference's test (tests/test_vllm_tp_placement.py:41-106 and on), both
ranks are built in ONE process -- ``tp_rank`` is an attribute vLLM's parameter base class reads
off the process group, overwritten per assertion -- and the assertion is always: what the ranks
hold, reassembled, equals the checkpoint.  Ramp-valued tensors make a misplacement a mismatch
at a nameable index.
"""

from __future__ import annotations

import pytest
import torch

pytest.importorskip("vllm", reason="the adapter needs vLLM to import")

TP = 2
IN_FEATURES = 2048
GROUP = 128


@pytest.fixture(scope="module", autouse=True)
def _parallel_state():
    """A world of one over gloo, only so vLLM's parameter base class can construct."""
    from conftest import vllm_world_of_one

    vllm_world_of_one()
    yield


def spec(bits, group_size=GROUP):
    from dynquant_b200.checkpoint import ModuleSpec

    return ModuleSpec(bits=bits, group_size=group_size)


def checkpoint_tensors(bits, rows, in_features=IN_FEATURES):
    from dynquant_b200.format import row_geometry

    g = row_geometry(bits, GROUP, in_features)
    words = torch.arange(rows * g.words_per_row, dtype=torch.int32).view(rows, g.words_per_row)
    scales = torch.arange(rows * g.num_groups, dtype=torch.float32).to(torch.bfloat16).view(rows, g.num_groups)
    return words, scales


def build(shards, partitions, in_per_partition=IN_FEATURES):
    from dynquant_b200.vllm_plugin import DynQuantLinearMethod

    layer = torch.nn.Module()
    DynQuantLinearMethod(None, shards).create_weights(
        layer, input_size_per_partition=in_per_partition, output_partition_sizes=list(partitions),
        input_size=IN_FEATURES, output_size=sum(partitions), params_dtype=torch.bfloat16, weight_loader=None)
    return layer


def set_rank(layer, rank):
    for name in ("qweight", "scales", "offsets"):
        param = getattr(layer, name)
        param.tp_rank, param.tp_size = rank, TP


def test_register_is_idempotent_and_the_config_parses():
    from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS, get_quantization_config

    from dynquant_b200.vllm_plugin import DynQuantConfig, register

    register()
    register()
    assert "dynquant" in QUANTIZATION_METHODS
    assert get_quantization_config("dynquant") is DynQuantConfig
    cfg = DynQuantConfig.from_config({
        "quant_method": "dynquant", "checkpoint_format": "dynquant-packed", "group_size": 128,
        "modules": {"model.layers.0.self_attn.q_proj": 4, "model.layers.0.self_attn.k_proj": {"bits": 2},
                    "model.layers.0.self_attn.v_proj": 3, "model.layers.0.mlp.experts.gate_up_proj": 3,
                    "model.layers.0.mlp.experts.down_proj": 4}})
    cfg.packed_modules_mapping = {"qkv_proj": ["q_proj", "k_proj", "v_proj"]}
    shards = cfg.resolve_shards("model.layers.0.self_attn.qkv_proj")
    assert [(n.rsplit(".", 1)[-1], s.bits) for n, s in shards] == [("q_proj", 4), ("k_proj", 2), ("v_proj", 3)]
    assert cfg.resolve_shards("model.layers.0.self_attn.o_proj") is None
    gate_up, down = cfg.resolve_expert_banks("model.layers.0.mlp.experts")
    assert (gate_up.bits, down.bits) == (3, 4)
    cfg.packed_modules_mapping = {"qkv_proj": ["q_proj", "k_proj", "x_proj"]}
    with pytest.raises(ValueError, match="all or none"):
        cfg.resolve_shards("model.layers.0.self_attn.qkv_proj")


def test_the_expert_layer_gets_a_method_instead_of_a_refusal():
    """The reference raises on vLLM's expert layer (integration/vllm_plugin/config.py:107-112);
    here its class is recognised the same way (by defining package) and given the MoE method."""
    from vllm.model_executor.layers.fused_moe.layer import FusedMoE
    from vllm.model_executor.layers.linear import LinearBase

    from dynquant_b200.vllm_plugin import DynQuantMoEMethod, is_fused_moe_class
    from vllm.model_executor.layers.fused_moe.fused_moe_method_base import FusedMoEMethodBase

    assert is_fused_moe_class(FusedMoE) and not is_fused_moe_class(LinearBase)
    assert issubclass(DynQuantMoEMethod, FusedMoEMethodBase)


def test_qkv_ranks_tile_the_checkpoint_rows():
    """q, k, v at three widths (256-, 192- and 512-word rows over the same input), two ranks."""
    widths = {"q": (4, 2048), "k": (3, 512), "v": (8, 512)}
    full = {n: checkpoint_tensors(b, r) for n, (b, r) in widths.items()}
    shards = [(f"l.{n}_proj", spec(b)) for n, (b, _) in widths.items()]
    for rank in range(TP):
        layer = build(shards, [r // TP for _, r in widths.values()])
        set_rank(layer, rank)
        offset = 0
        for shard_id, (name, (_, rows)) in enumerate(widths.items()):
            size = rows // TP
            for attr, source in (("qweight", full[name][0]), ("scales", full[name][1])):
                getattr(layer, attr).load_qkv_weight(loaded_weight=source, shard_offset=offset, shard_size=size,
                                                     shard_id=name, num_heads=1)
            offset += size
            g = layer.dynquant_geometry
            assert torch.equal(g.view_qweight(layer.qweight.data, shard_id), full[name][0][rank * size:(rank + 1) * size])
            assert torch.equal(g.view_scale(layer.scales.data, shard_id), full[name][1][rank * size:(rank + 1) * size])


def test_replicated_kv_heads_read_the_same_rows_on_every_rank():
    k_rows = 128
    k_words, k_scales = checkpoint_tensors(4, k_rows)
    shards = [("l.q_proj", spec(4)), ("l.k_proj", spec(4))]
    held = []
    for rank in range(TP):
        layer = build(shards, [1024, k_rows])
        set_rank(layer, rank)
        for attr, source in (("qweight", k_words), ("scales", k_scales)):
            getattr(layer, attr).load_qkv_weight(loaded_weight=source, shard_offset=1024, shard_size=k_rows,
                                                 shard_id="k", num_heads=TP)
        held.append(layer.dynquant_geometry.view_qweight(layer.qweight.data, 1).clone())
    assert torch.equal(held[0], k_words) and torch.equal(held[0], held[1])


def test_merged_column_ranks_tile_the_checkpoint_rows():
    gate, up = checkpoint_tensors(4, 4096), checkpoint_tensors(3, 4096)
    shards = [("l.gate_proj", spec(4)), ("l.up_proj", spec(3))]
    for rank in range(TP):
        layer = build(shards, [2048, 2048])
        set_rank(layer, rank)
        for shard_id, (source, offset) in enumerate(((gate, 0), (up, 2048))):
            layer.qweight.load_merged_column_weight(loaded_weight=source[0], shard_offset=offset, shard_size=2048)
            got = layer.dynquant_geometry.view_qweight(layer.qweight.data, shard_id)
            assert torch.equal(got, source[0][rank * 2048:(rank + 1) * 2048])


def test_column_parallel_ranks_tile_the_rows():
    words, scales = checkpoint_tensors(2, 1024)
    parts = []
    for rank in range(TP):
        layer = build([("l.up", spec(2))], [512])
        set_rank(layer, rank)
        layer.qweight.load_column_parallel_weight(words)
        parts.append(layer.dynquant_geometry.view_qweight(layer.qweight.data, 0).clone())
    assert torch.equal(torch.cat(parts), words)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_input_sharded_ranks_tile_the_word_axis(bits):
    """o_proj / down_proj: every row, this rank's words -- only legal on a group boundary, and the
    words per group differ by width (3-bit packs 32 values into 3 words)."""
    rows = 1024
    words, scales = checkpoint_tensors(bits, rows)
    halves, scale_halves = [], []
    for rank in range(TP):
        layer = build([("l.o_proj", spec(bits))], [rows], in_per_partition=IN_FEATURES // TP)
        assert layer.dynquant_row_split is not None
        set_rank(layer, rank)
        layer.qweight.load_row_parallel_weight(words)
        layer.scales.load_row_parallel_weight(scales)
        g = layer.dynquant_geometry
        halves.append(g.view_qweight(layer.qweight.data, 0).clone())
        scale_halves.append(g.view_scale(layer.scales.data, 0).clone())
    assert torch.equal(torch.cat(halves, dim=1), words)
    assert torch.equal(torch.cat(scale_halves, dim=1), scales)


def test_illegal_input_splits_are_refused_when_the_layer_is_built():
    from dynquant_b200.vllm_plugin import DynQuantLinearMethod

    three_groups = 3 * GROUP  # three groups over two ranks
    with pytest.raises(ValueError, match="down_proj"):
        DynQuantLinearMethod(None, [("l.down_proj", spec(4))]).create_weights(
            torch.nn.Module(), input_size_per_partition=three_groups // TP, output_partition_sizes=[512],
            input_size=three_groups, output_size=512, params_dtype=torch.bfloat16, weight_loader=None)
    with pytest.raises(ValueError, match="more than one"):
        DynQuantLinearMethod(None, [("l.a", spec(4)), ("l.b", spec(3))]).create_weights(
            torch.nn.Module(), input_size_per_partition=IN_FEATURES // TP, output_partition_sizes=[256, 256],
            input_size=IN_FEATURES, output_size=512, params_dtype=torch.bfloat16, weight_loader=None)


def test_a_tensor_of_the_wrong_width_is_refused_not_copied():
    words3, _ = checkpoint_tensors(3, 512)
    layer = build([("l.up", spec(4))], [512])
    set_rank(layer, 0)
    layer.qweight.tp_size = 1
    with pytest.raises(ValueError, match="different runs"):
        layer.qweight.load_column_parallel_weight(words3)


def test_expert_bank_loader_places_whole_banks_and_single_experts():
    from dynquant_b200.vllm_plugin import _bank_loader

    experts, inter, words = 4, 8, 6
    bank = torch.nn.Parameter(torch.zeros(experts, 2 * inter, words, dtype=torch.int32), requires_grad=False)
    whole = torch.arange(experts * 2 * inter * words, dtype=torch.int32).view(experts * 2 * inter, words)
    _bank_loader(bank, whole)
    assert torch.equal(bank.data.view(-1, words), whole)
    gate = torch.full((inter, words), 7, dtype=torch.int32)
    up = torch.full((inter, words), 9, dtype=torch.int32)
    _bank_loader(bank, gate, "experts.2.gate_proj.qweight", "w1", 2)
    _bank_loader(bank, up, "experts.2.up_proj.qweight", "w3", 2)
    assert torch.equal(bank.data[2, :inter], gate) and torch.equal(bank.data[2, inter:], up)
    assert torch.equal(bank.data[1].reshape(-1, words), whole[2 * inter:4 * inter])
    with pytest.raises(ValueError):
        _bank_loader(bank, gate[:, :3].contiguous(), "experts.0.gate_proj.qweight", "w1", 0)
