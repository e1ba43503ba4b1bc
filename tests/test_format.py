"""The host-side format layer (``dynquant_b200.format``) against the oracle and the golden
vectors: geometry, bit packing, the QuantTensor container.  No GPU."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import raw
from dynquant_b200 import PackingError, QuantTensor, pack_nbit, row_geometry, unpack_nbit
from oracle import oracle as O

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "golden_v1.npz")


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("n", [1, 2, 3, 7, 8, 31, 32, 33, 37, 96, 127, 128, 129, 1023])
def test_pack_is_a_bijection_and_matches_reference_words(bits, n):
    codes = torch.from_numpy(GOLDEN[f"pack_b{bits}_n{n}_codes"].astype(np.int64))
    words = pack_nbit(codes, bits)
    assert words.dtype == torch.int32
    assert (raw(words) == GOLDEN[f"pack_b{bits}_n{n}_words"]).all()
    assert torch.equal(unpack_nbit(words, bits, n).to(torch.int64), codes)


def test_rank3_and_extremal_codes():
    for bits in (2, 3, 4, 8):
        q = torch.full((2, 3, 70), (1 << bits) - 1)
        words = pack_nbit(q, bits)
        assert words.shape[:2] == (2, 3)
        assert torch.equal(unpack_nbit(words, bits, 70).to(torch.int64), q)  # sign bit of int32 in play
        assert (raw(words) == O.c_pack(q.numpy().astype(np.uint8), bits)).all()


def test_out_of_range_codes_and_bad_geometry_are_rejected():
    with pytest.raises(PackingError):
        pack_nbit(torch.tensor([[4]]), 2)
    with pytest.raises(PackingError):
        pack_nbit(torch.tensor([[0]]), 5)
    with pytest.raises(PackingError):
        row_geometry(4, 48, 512)  # not a multiple of 32
    with pytest.raises(PackingError):
        unpack_nbit(torch.zeros(1, 3, dtype=torch.int32), 4, 64)


def test_per_row_geometry_table():
    # docs/format-spec.md:256-262
    for k, bits, words in ((4, 2, 1), (4, 4, 1), (4, 8, 1), (100, 4, 13), (5120, 3, 480)):
        g = row_geometry(bits, -1, k)
        assert (g.num_groups, g.words_per_group, g.effective_group, g.padded_in_features) == (1, words, k, k)
    g = row_geometry(3, 128, 320)
    assert (g.num_groups, g.padded_in_features, g.words_per_row) == (3, 384, 36)


@pytest.mark.parametrize("ci", range(len([k for k in GOLDEN.files if k.endswith("_spec")])))
def test_from_dense_reproduces_the_reference_encoder(ci):
    rows, k, group, bits, m, with_off = (int(v) for v in GOLDEN[f"case{ci}_spec"])
    meta = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[str(GOLDEN[f"case{ci}_meta"])]
    qt = QuantTensor.from_dense(torch.from_numpy(GOLDEN[f"case{ci}_dense"]), bits=bits, group_size=group,
                                compute_dtype=meta)
    qt.validate()
    assert (raw(qt.packed) == GOLDEN[f"case{ci}_packed"]).all()
    assert (raw(qt.scales) == GOLDEN[f"case{ci}_scales"]).all()
    if with_off:
        assert (raw(qt.offsets) == GOLDEN[f"case{ci}_offsets"]).all()


def test_stacked_experts_fold_to_rows_and_rows_are_independent():
    torch.manual_seed(0)
    bank = torch.randn(3, 8, 256)
    qt = QuantTensor.from_dense(bank, bits=4, group_size=128)
    assert qt.num_rows == 24 and qt.logical_shape == (3, 8, 256)
    one = QuantTensor.from_dense(bank[1], bits=4, group_size=128)
    part = qt.rows(8, 16)
    assert torch.equal(part.packed, one.packed) and torch.equal(part.scales, one.scales)
    assert part.row_offset == 8


def test_nbytes_counts_metadata():
    qt = QuantTensor.from_dense(torch.randn(256, 512), bits=3, group_size=128)
    assert qt.nbytes == 53248  # docs/format-spec.md:661


def test_constant_group_is_exact():
    w = torch.full((2, 128), 0.375)
    qt = QuantTensor.from_dense(w, bits=2, group_size=128)
    assert float(qt.scales.abs().max()) == 0.0 and float(qt.offsets[0, 0]) == 0.375
    assert int(qt.packed.abs().max()) == 0


def test_linear_method_accepts_an_input_slice_on_group_boundaries_only():
    """Row-parallel placement: the layer's buffers are sized for this rank's slice of the input
    axis; a slice that cuts a group is refused (reference serving_common/geometry.py:481-551)."""
    import pytest
    import torch

    from dynquant_b200.plugin import DynQuantLinearMethod, ShardSpec

    method = DynQuantLinearMethod(None, [ShardSpec("down_proj", 3, 128, 64)])
    layer = torch.nn.Module()
    method.create_weights(layer, 256, [64], 512, 64, torch.float16)  # half of a 512-wide input
    assert layer.qweight.numel() == 64 * (256 * 3 // 32) and layer.scales.numel() == 64 * 2
    with pytest.raises(ValueError, match="whole number of groups"):
        method.create_weights(torch.nn.Module(), 192, [64], 384, 64, torch.float16)
