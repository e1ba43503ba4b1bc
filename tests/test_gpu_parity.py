"""CUDA kernels against the CPU oracle, through the C ABI.

Geometry list, activation-row list, seeds and tolerances are those of the
reference's own parity suite (tests/test_kernels_parity.py:50-68, :98-120,
:172-203, :206-229, :307-353), restated against this library:

* dequant is compared bit for bit (integer work, one rounding);
* gemv is compared on the fp32 accumulators to 1e-3 (normwise and max/max)
  against ``x.float() @ dequant(fp32).T`` and the 16-bit output to one ulp of
  the rounded oracle.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import TAG, from_raw, make_quant, raw

pytestmark = pytest.mark.gpu

PER_ROW = -1
GEOMETRIES = [
    (128, 512, 128),
    (70, 2048, 128),
    (64, 320, 128),
    (33, 256, 128),
    (16, 128, 32),
    (48, 100, PER_ROW),
    (7, 4, PER_ROW),
    (72, 4304, 128),
    (80, 2048, 128),
    (65, 3072, 128),
    (40, 1024, 64),
    (24, 768, 64),
]
BITS = [2, 3, 4, 8]


def oracle_geom(qt):
    from oracle import oracle as O

    return O.geometry(qt.bits, qt.group_size, qt.in_features)


def oracle_dequant(qt, out_dtype=None):
    from oracle import oracle as O

    tag = TAG[qt.scales.dtype]
    return O.c_dequant(raw(qt.packed), raw(qt.scales), raw(qt.offsets), tag, oracle_geom(qt),
                       TAG[out_dtype or qt.scales.dtype])


def oracle_gemv(x, qt):
    from oracle import oracle as O

    return O.c_gemv(raw(x), TAG[x.dtype], raw(qt.packed), raw(qt.scales), raw(qt.offsets),
                    TAG[qt.scales.dtype], oracle_geom(qt))


def bits_equal(got: torch.Tensor, want_raw: np.ndarray) -> bool:
    g = raw(got)
    if g.dtype == np.float32:
        return bool((g.view(np.uint32) == want_raw.view(np.uint32)).all())
    return bool((g == want_raw).all())


def within_one_ulp_16(got: torch.Tensor, want32: np.ndarray, slack: float = 2e-5) -> bool:
    """``got`` (fp16/bf16) is the fp32 oracle rounded once, give or take one unit in the last
    place -- plus ``slack * max|oracle|`` of absolute room, because an output that nearly
    cancels to zero has an ulp far below the fp32 accumulation noise of either side."""
    want = torch.from_numpy(want32)
    rounded = want.to(got.dtype)
    mant = 10 if got.dtype == torch.float16 else 7
    ulp = torch.maximum(rounded.float().abs(), torch.tensor(6e-5)) * 2.0 ** (-mant)
    err = (got.float().cpu() - rounded.float()).abs()
    return bool((err <= ulp + slack * float(want.abs().max())).all())


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize(("rows", "k", "group"), GEOMETRIES)
def test_dequant_is_bit_exact(bits, rows, k, group):
    from dynquant_b200 import ops

    qt = make_quant(rows, k, group, bits, torch.float16).to("cuda")
    got = ops.dequant(qt.packed, qt.scales, qt.offsets, bits, qt.geometry.effective_group, k)
    assert got.shape == (rows, k) and got.dtype == torch.float16
    assert bits_equal(got, oracle_dequant(qt))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bits", BITS)
def test_dequant_every_compute_dtype(bits, dtype):
    from dynquant_b200 import ops

    qt = make_quant(64, 256, 128, bits, dtype).to("cuda")
    got = ops.dequant(qt.packed, qt.scales, qt.offsets, bits, 128, 256)
    assert got.dtype == dtype
    assert bits_equal(got, oracle_dequant(qt))


@pytest.mark.parametrize("bits", BITS)
def test_dequant_without_offsets(bits):
    from dynquant_b200 import ops

    qt = make_quant(64, 256, 128, bits, torch.float16, with_offsets=False).to("cuda")
    got = ops.dequant(qt.packed, qt.scales, None, bits, 128, 256)
    assert bits_equal(got, oracle_dequant(qt))


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize(("rows", "k", "group"), GEOMETRIES)
def test_gemv_matches_dequant_then_matmul(m, bits, rows, k, group):
    from dynquant_b200 import ops

    qt = make_quant(rows, k, group, bits, torch.float16).to("cuda")
    gen = torch.Generator().manual_seed(m)
    x = torch.randn(m, k, generator=gen).to(torch.float16).cuda()
    want = oracle_gemv(x, qt)
    args = (x, qt.packed, qt.scales, qt.offsets, bits, qt.geometry.effective_group, k)

    acc = ops.gemv(*args, out_dtype=torch.float32).cpu().numpy()
    assert acc.shape == (m, rows)
    scale = np.abs(want).max() + 1e-30
    assert np.abs(acc - want).max() / scale <= 1e-3
    assert np.linalg.norm(acc - want) / (np.linalg.norm(want) + 1e-30) <= 1e-3

    got = ops.gemv(*args)
    assert got.dtype == torch.float16 and got.shape == (m, rows)
    # the 16-bit output is the fp32 accumulator rounded once
    assert torch.equal(got.cpu(), torch.from_numpy(acc).to(torch.float16))
    assert within_one_ulp_16(got, want)
    torch.testing.assert_close(got.float().cpu(), torch.from_numpy(want), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("meta", [torch.float16, torch.bfloat16])
def test_gemv_mixed_dtypes(bits, meta):
    """bf16 activations against fp16 (or bf16) scales: the pair BASELINE's first config asks for."""
    from dynquant_b200 import ops

    qt = make_quant(96, 2048, 128, bits, meta).to("cuda")
    x = torch.randn(1, 2048, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
    want = oracle_gemv(x, qt)
    acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, 128, 2048, out_dtype=torch.float32).cpu().numpy()
    assert np.abs(acc - want).max() / np.abs(want).max() <= 1e-3
    got = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, 128, 2048)
    assert got.dtype == torch.bfloat16
    assert within_one_ulp_16(got, want)


def test_gemv_is_deterministic():
    from dynquant_b200 import ops

    qt = make_quant(512, 1024, 128, 3, torch.float16).to("cuda")
    x = torch.randn(4, 1024, dtype=torch.float16, device="cuda")
    args = (x, qt.packed, qt.scales, qt.offsets, 3, 128, 1024)
    first = ops.gemv(*args)
    for _ in range(8):
        assert torch.equal(ops.gemv(*args), first)


def test_gemv_refuses_more_rows_than_it_was_built_for():
    from dynquant_b200 import ops

    qt = make_quant(64, 256, 128, 4, torch.float16).to("cuda")
    x = torch.randn(ops.gemv_max_rows() + 1, 256, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="exceeds the kernel's limit"):
        ops.gemv(x, qt.packed, qt.scales, qt.offsets, 4, 128, 256)


def test_unresolved_per_row_sentinel_is_rejected():
    from dynquant_b200 import ops

    qt = make_quant(48, 100, PER_ROW, 3, torch.float16).to("cuda")
    with pytest.raises(RuntimeError, match="resolved positive count"):
        ops.dequant(qt.packed, qt.scales, qt.offsets, 3, PER_ROW, 100)


def test_mismatched_scales_are_rejected():
    from dynquant_b200 import ops

    qt = make_quant(64, 256, 128, 4, torch.float16).to("cuda")
    with pytest.raises(RuntimeError):
        ops.dequant(qt.packed, qt.scales[:-1], qt.offsets[:-1], 4, 128, 256)


def test_torch_ops_namespace_runs_the_cuda_kernels():
    import dynquant_b200  # noqa: F401  (registers torch.ops.dynquant)

    qt = make_quant(128, 512, 128, 4, torch.float16).to("cuda")
    x = torch.randn(2, 512, dtype=torch.float16, device="cuda")
    got = torch.ops.dynquant.gemv(x, qt.packed, qt.scales, qt.offsets, 4, 128, 512)
    want = oracle_gemv(x, qt)
    torch.testing.assert_close(got.float().cpu(), torch.from_numpy(want), rtol=2e-2, atol=2e-2)
    dense = torch.ops.dynquant.dequant(qt.packed, qt.scales, qt.offsets, 4, 128, 512)
    assert bits_equal(dense, oracle_dequant(qt))
    assert int(torch.ops.dynquant.abi_version()) == 2
    assert int(torch.ops.dynquant.gemv_max_rows()) == 8
    with pytest.raises(RuntimeError):
        torch.ops.dynquant.gemv(x.cpu(), qt.packed.cpu(), qt.scales.cpu(), qt.offsets.cpu(), 4, 128, 512)


def test_empty_shapes_return_empty():
    from dynquant_b200 import ops

    qt = make_quant(64, 256, 128, 4, torch.float16).to("cuda")
    x = torch.empty(0, 256, dtype=torch.float16, device="cuda")
    assert ops.gemv(x, qt.packed, qt.scales, qt.offsets, 4, 128, 256).shape == (0, 64)
    empty = qt.rows(0, 0)
    assert ops.dequant(empty.packed, empty.scales, empty.offsets, 4, 128, 256).shape == (0, 256)


# ---- regimes of the tiled tensor-core kernel (persistent CTAs, 64-value groups, fused shards,
# ---- activation-row split): same oracle, same bar


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("group", [64, 128])
def test_gemv_many_short_rows_take_the_persistent_regime(bits, group):
    """64,000 rows of 256 values: more row tiles than one wave of CTAs holds, so CTAs walk over
    several items through their ring; with 64-value groups this is the only tensor-core kernel."""
    from dynquant_b200 import ops

    rows, k = 64000, 256
    qt = make_quant(rows, k, group, bits, torch.float16).to("cuda")
    for m in (1, 8):
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(bits + m)).to(torch.bfloat16).cuda()
        want = oracle_gemv(x, qt)
        acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, qt.geometry.effective_group, k,
                       out_dtype=torch.float32).cpu().numpy()
        assert np.abs(acc - want).max() / (np.abs(want).max() + 1e-30) <= 1e-3
        assert np.linalg.norm(acc - want) / (np.linalg.norm(want) + 1e-30) <= 1e-3


@pytest.mark.parametrize("group", [64, 128])
def test_fused_shards_of_every_width_in_one_launch(group):
    """Four shards (2, 3, 4, 8 bits) against one activation: one launch, each CTA the body of
    its shard's width, bias folded into the store."""
    from dynquant_b200 import ops

    k = 1024
    sizes = [(2, 96), (3, 160), (4, 33), (8, 64)]
    shards = [make_quant(rows, k, group, bits, torch.float16, seed=40 + bits).to("cuda") for bits, rows in sizes]
    total = sum(rows for _, rows in sizes)
    bias = torch.randn(total, generator=torch.Generator().manual_seed(7)).to(torch.float32).cuda()
    for m in (1, 5):
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(torch.bfloat16).cuda()
        before = ops.launch_count()
        got = ops.gemv_shards(x, shards, bias, out_dtype=torch.float32)
        assert ops.launch_count() - before == 1
        want = np.concatenate([oracle_gemv(x, qt) for qt in shards], axis=1) + bias.cpu().numpy()
        assert got.shape == (m, total)
        assert np.abs(got.cpu().numpy() - want).max() / np.abs(want).max() <= 1e-3


@pytest.mark.parametrize("bits", [3, 8])
def test_gemv_splits_activation_rows_when_their_fragments_do_not_fit(bits):
    """8 rows x 14336 values of staged fragments exceed shared memory (at 8 bits even 4 do): the
    rows are processed in halves, on the tensor-core path, with the same results."""
    from dynquant_b200 import ops

    rows, k, m = 64, 14336, 8
    qt = make_quant(rows, k, 128, bits, torch.float16).to("cuda")
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    want = oracle_gemv(x, qt)
    acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, 128, k, out_dtype=torch.float32).cpu().numpy()
    assert np.abs(acc - want).max() / np.abs(want).max() <= 1e-3
    single = torch.cat([ops.gemv(x[i : i + 1], qt.packed, qt.scales, qt.offsets, bits, 128, k, out_dtype=torch.float32)
                        for i in range(m)])
    assert np.abs(acc - single.cpu().numpy()).max() / np.abs(want).max() <= 1e-5


def test_bandwidth_probes_touch_every_byte():
    """``dq_probe_read`` XORs every 32-bit word of the buffer; ``dq_probe_copy`` is a copy.

    They are the denominators of a bandwidth fraction (the reference measures the same pair
    with ``sum()`` and ``copy_``, commands/bench.py:95-120): a probe that skipped a byte would
    overstate the achievable bandwidth.
    """
    from dynquant_b200 import ops

    gen = torch.Generator().manual_seed(17)
    for words in (4, 1024 + 4, 3 * 1_000_003 * 4 + 8):  # tails shorter than one unrolled round, ragged sizes
        host = torch.randint(-(2**31), 2**31 - 1, (words,), dtype=torch.int32, generator=gen)
        buf = host.cuda()
        sink = torch.zeros(1, dtype=torch.int64, device="cuda")
        ops.probe_read(buf, sink)
        expect = int(np.bitwise_xor.reduce(host.numpy().view(np.uint32)))
        assert int(sink.item()) & 0xFFFFFFFF == expect
        dst = torch.zeros_like(buf)
        ops.probe_copy(dst, buf)
        assert torch.equal(dst.cpu(), host)
    with pytest.raises(RuntimeError, match="multiple of 16 bytes"):
        ops.probe_read(torch.zeros(3, dtype=torch.int32, device="cuda"), sink)
    with pytest.raises(RuntimeError, match="overlap"):
        ops.probe_copy(buf[4:12], buf[8:16])
