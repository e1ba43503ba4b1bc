"""Host logic of the packed modules (no device needed): buffers, tied tables, cached views.

Restates the CPU half of the reference's module tests (tests/test_runtime_linear.py:114-120 state
dict keys, :136-185 tied tables share one buffer and follow it when the storage moves)."""

from __future__ import annotations

import pytest
import torch

from conftest import make_quant


def test_state_dict_keys_and_attributes():
    from dynquant_b200.runtime import DynQuantEmbedding, DynQuantLinear

    qt = make_quant(48, 256, 128, 3, torch.float16)
    lin = DynQuantLinear(qt, torch.zeros(48, dtype=torch.float16))
    assert set(lin.state_dict()) == {"qweight", "scales", "offsets", "bias"}
    assert (lin.bits, lin.group_size, lin.in_features, lin.out_features) == (3, 128, 256, 48)
    assert "3-bit" in repr(lin)
    emb = DynQuantEmbedding(qt, padding_idx=0)
    assert (emb.num_embeddings, emb.embedding_dim, emb.padding_idx) == (48, 256, 0)
    assert set(emb.state_dict()) == {"qweight", "scales", "offsets"}
    assert DynQuantLinear(qt).bias is None


def test_tied_table_is_held_once_and_followed_when_the_storage_moves():
    from dynquant_b200.runtime import DynQuantEmbedding, DynQuantLinear, packed_bytes

    qt = make_quant(64, 128, -1, 4, torch.float16)
    model = torch.nn.Module()
    model.embed = DynQuantEmbedding(qt)
    model.head = DynQuantLinear(qt, tied_to=model.embed)
    assert model.head.holder is model.embed
    assert sorted(model.state_dict()) == ["embed.offsets", "embed.qweight", "embed.scales"]  # the table, once
    assert packed_bytes(model) == qt.nbytes
    before = model.head.weight_qt
    assert model.head.weight_qt is before  # the view is cached, not rebuilt per call
    # what `.to(device)` does to a module: every buffer replaced by a new tensor
    model._apply(lambda t: t.clone())
    after = model.head.weight_qt
    assert after is not before
    assert after.packed.data_ptr() == model.embed.qweight.data_ptr()
    assert torch.equal(after.packed, qt.packed) and torch.equal(after.scales, qt.scales)


def test_only_matrices_in_the_linear_layout_are_accepted():
    from dataclasses import replace

    from dynquant_b200.runtime import DynQuantLinear

    qt = make_quant(16, 128, 128, 4, torch.float16)
    with pytest.raises(ValueError):
        DynQuantLinear(replace(qt, logical_shape=(2, 8, 128)))
    with pytest.raises(NotImplementedError):
        DynQuantLinear(replace(qt, layout="tc_shuffled"))
