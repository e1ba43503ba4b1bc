"""Parity at the benchmark configurations' own shapes, per kernel, and with guarded buffers.

Same oracle and bars as ``test_gpu_parity.py`` (fp32 accumulators within 1e-3 of
``x.float() @ dequant(fp32).T``, normwise and max/max).  What this file adds:

* every tensor-core kernel is reached on purpose, and ``dq_last_kernel`` proves which one ran;
* BASELINE's first configuration exactly, the corner shapes of its width/shape sweep, and the
  248,320-row head of its decode stack;
* canary-padded output buffers on every tail geometry: a store outside ``out`` fails the test
  (the stand-in for a memory checker, which this pool does not offer);
* the two SIMT paths against each other, the selection made by an environment variable in a
  child process (reference tests/test_kernels_parity.py:232-304).
"""

from __future__ import annotations

import ctypes
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

from conftest import ROOT, make_quant
from test_gpu_parity import GEOMETRIES, oracle_dequant, oracle_gemv, within_one_ulp_16

pytestmark = pytest.mark.gpu

BITS = [2, 3, 4, 8]


def random_qt(rows, k, bits, group=128, meta=torch.float16, seed=0, offsets=True):
    """Uniform random codes, U(0.005, 0.02) scales, offsets -2^(b-1) * scale: the benchmark's data."""
    from dynquant_b200.workloads import random_quant_tensor

    gen = torch.Generator(device="cuda").manual_seed(seed)
    qt = random_quant_tensor(rows, k, bits, group_size=group, meta_dtype=meta, device="cuda", generator=gen)
    if not offsets:
        qt.offsets = None
    return qt


def check_acc(acc: torch.Tensor, want: np.ndarray, tol: float = 1e-3) -> None:
    got = acc.float().cpu().numpy()
    assert got.shape == want.shape
    scale = np.abs(want).max() + 1e-30
    assert np.abs(got - want).max() / scale <= tol
    assert np.linalg.norm(got - want) / (np.linalg.norm(want) + 1e-30) <= tol


# ---- (a) the streaming kernel: long matrices, every width -------------------------------------


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize(("rows", "k", "m", "xdt", "meta", "offsets"), [
    (19001, 512, 1, torch.bfloat16, torch.float16, True),    # rows not a multiple of 16
    (19001, 512, 8, torch.bfloat16, torch.float16, True),
    (20480, 512, 3, torch.float16, torch.bfloat16, False),   # fp16 x, bf16 scales, no offsets
    (24000, 2048, 1, torch.bfloat16, torch.bfloat16, True),
    (33000, 512, 8, torch.float16, torch.float16, True),
])
def test_long_matrices_take_the_streaming_kernel(bits, rows, k, m, xdt, meta, offsets):
    from dynquant_b200 import ops

    qt = random_qt(rows, k, bits, meta=meta, seed=bits * 31 + rows, offsets=offsets)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(m + bits)).to(xdt).cuda()
    args = (x, qt.packed, qt.scales, qt.offsets, bits, 128, k)
    acc = ops.gemv(*args, out_dtype=torch.float32)
    assert ops.last_kernel() == "gemv_mma_stream_kernel"
    want = oracle_gemv(x, qt)
    check_acc(acc, want)
    got = ops.gemv(*args)
    assert torch.equal(got.cpu(), acc.cpu().to(xdt))  # the 16-bit output is the accumulator rounded once
    assert within_one_ulp_16(got, want)
    assert torch.equal(ops.gemv(*args), got)  # bit-identical repeat


@pytest.mark.parametrize("bits", BITS)
def test_the_register_ring_kernel_takes_what_the_other_two_refuse(bits):
    """A long matrix whose step count is odd (K = 384: three steps) fits neither the streaming
    kernel (whole blocks of steps) nor the tiled one (long, one matrix): gemv_mma_kernel."""
    from dynquant_b200 import ops

    rows, k = 19200, 384
    qt = random_qt(rows, k, bits, seed=bits)
    x = torch.randn(2, k, generator=torch.Generator().manual_seed(bits)).to(torch.bfloat16).cuda()
    acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, 128, k, out_dtype=torch.float32)
    assert ops.last_kernel() == "gemv_mma_kernel"
    check_acc(acc, oracle_gemv(x, qt))


# ---- (b) BASELINE configuration 1, exactly ------------------------------------------------------


@pytest.mark.parametrize("meta", [torch.float16, torch.bfloat16])
def test_baseline_config_1(meta):
    """M=1, K=2048, N=6144, 4-bit, groups of 128, codes uniform in [0, 15], scales U(0.005, 0.02),
    zero-point 8 written out as offsets = -8 * scale, bf16 activations ~ N(0, 1)."""
    from dynquant_b200 import ops

    qt = random_qt(6144, 2048, 4, meta=meta, seed=1)
    assert torch.equal(qt.offsets.float(), (-8.0 * qt.scales.float()).to(meta).float())
    x = torch.randn(1, 2048, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, 4, 128, 2048, out_dtype=torch.float32)
    assert ops.last_kernel() == "gemv_mma_tile_kernel"
    want = oracle_gemv(x, qt)
    check_acc(acc, want)
    got = ops.gemv(x, qt.packed, qt.scales, qt.offsets, 4, 128, 2048)
    assert got.dtype == torch.bfloat16 and within_one_ulp_16(got, want)
    dense = ops.dequant(qt.packed, qt.scales, qt.offsets, 4, 128, 2048)
    assert (dense.cpu().view(torch.int16).numpy().view(np.uint16) == oracle_dequant(qt)).all()


# ---- (c) corners of the width / shape sweep (configuration 5) -----------------------------------

SWEEP_SHAPES = [(14336, 4096), (4096, 14336), (4096, 4096), (4097, 4096)]  # (rows N, reduction K)


@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("shape", range(len(SWEEP_SHAPES)))
def test_sweep_shapes(bits, group, shape):
    """Every (width, group, shape) of the sweep; the activation-row counts 1, 4 and 16 rotate over
    the combinations (16 rows go through quantized_matmul's chunks of 8)."""
    from dynquant_b200 import ops

    rows, k = SWEEP_SHAPES[shape]
    m = (1, 4, 16)[(shape + bits + group // 64) % 3]
    qt = random_qt(rows, k, bits, group=group, seed=bits * 7 + shape)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(shape)).to(torch.bfloat16).cuda()
    want = oracle_gemv(x, qt)
    if m <= ops.gemv_max_rows():
        acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, group, k, out_dtype=torch.float32)
        assert ops.last_kernel().startswith(("gemv_mma", "gemv_rows"))  # a tensor-core kernel, not the SIMT fallback
    else:
        acc = ops.gemv_row_chunks(x, [qt], out_dtype=torch.float32)
    check_acc(acc, want)
    out = ops.quantized_matmul(x, qt)
    assert out.dtype == torch.bfloat16 and within_one_ulp_16(out, want)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("m,group", [(9, 128), (16, 128), (20, 128), (32, 128), (33, 128), (40, 128), (64, 128),
                                     (9, 64), (16, 64), (17, 64), (40, 64)])
def test_many_rows_on_a_large_matrix_take_one_pass_over_the_weights(m, group, bits):
    """The many-rows kernel (matrices with a CTA for most SMs): the fragments of a step decoded once
    and fed to up to four column blocks of eight activation rows; one launch per 32 rows (per 16
    with 64-value groups: two accumulators per column block), every row against the oracle."""
    from dynquant_b200 import _lib, ops

    meta = torch.bfloat16 if (m + bits) % 2 else torch.float16
    qt = random_qt(12809, 1024, bits, group=group, meta=meta, seed=m, offsets=bits != 3)  # a ragged row count
    act = torch.float16 if m % 3 == 0 else torch.bfloat16
    x = torch.randn(m, 1024, generator=torch.Generator().manual_seed(m)).to(act).cuda()
    before = int(_lib.load().dq_launch_count())
    acc = ops.gemv_row_chunks(x, [qt], out_dtype=torch.float32)
    per_launch = 32 if group == 128 else 16
    assert int(_lib.load().dq_launch_count()) - before == (m + per_launch - 1) // per_launch
    assert ops.last_kernel() == "gemv_rows_kernel"
    want = oracle_gemv(x, qt)
    check_acc(acc, want)
    out = ops.quantized_matmul(x, qt)
    assert out.dtype == act and within_one_ulp_16(out, want)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("rows,k,m,group", [(2048, 6144, 16, 128), (4096 + 5, 14336, 9, 128), (3072, 8192, 40, 128),
                                            (8192, 8192, 64, 128), (6144, 4096, 33, 128),
                                            (2048, 6144, 16, 64), (4096 + 5, 14336, 9, 64), (3072, 8192, 24, 64)])
def test_many_rows_on_a_matrix_with_few_rows_slice_the_reduction_axis(rows, k, m, group, bits):
    """Matrices with too few rows for a CTA per SM (down-projections): the many-rows kernel's CTAs
    of one row group form a thread-block cluster that slices the reduction axis; the slices' sums
    are added in slice order by the cluster's first CTA -- every row against the oracle, and the
    same bits on a second run."""
    from dynquant_b200 import _lib, ops

    meta = torch.bfloat16 if (m + bits) % 2 else torch.float16
    qt = random_qt(rows, k, bits, group=group, meta=meta, seed=m + bits, offsets=bits != 2)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(torch.bfloat16).cuda()
    before = int(_lib.load().dq_launch_count())
    acc = ops.gemv_row_chunks(x, [qt], out_dtype=torch.float32)
    per_launch = 32 if group == 128 else 16
    assert int(_lib.load().dq_launch_count()) - before == (m + per_launch - 1) // per_launch
    assert ops.last_kernel() == "gemv_rows_kernel"
    check_acc(acc, oracle_gemv(x, qt))
    again = ops.gemv_row_chunks(x, [qt], out_dtype=torch.float32)
    assert torch.equal(acc, again)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("rows,k,m,group", [(1536, 8960, 1, 128), (1536 + 3, 8960, 8, 128), (2048, 11008, 3, 128),
                                            (4096, 14336, 8, 128), (4096, 14336, 6, 128),
                                            (1536 + 3, 8960, 5, 64), (2048, 11008, 1, 64), (4096, 14336, 8, 64)])
def test_matrices_the_tiled_kernel_is_a_poor_fit_for_take_the_many_rows_kernel(rows, k, m, group, bits):
    """One to eight activation rows: step counts with few factors of two (70 and 86 steps -- blocks
    of two steps at the low widths) on matrices of few rows, and six to eight rows x a long reduction
    axis (the staged activation would fill the tiled kernel's shared memory).  Against the oracle,
    with a bias, through the operator (16-bit output = the accumulator rounded once)."""
    from dynquant_b200 import ops

    meta = torch.float16 if (m + bits) % 2 else torch.bfloat16
    act = torch.float16 if m == 3 else torch.bfloat16
    qt = random_qt(rows, k, bits, group=group, meta=meta, seed=m * 10 + bits, offsets=bits != 8)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(act).cuda()
    bias = torch.randn(rows, generator=torch.Generator().manual_seed(7)).to(act).cuda()
    cluster_kernels = ("gemv_rows_kernel", "gemv_mma_stream_sliced_kernel")  # (the second: from 16 MB on, 128-value groups)
    acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, group, k, out_dtype=torch.float32)
    assert ops.last_kernel() in cluster_kernels
    want = oracle_gemv(x, qt)
    check_acc(acc, want)
    out = ops.gemv_shards(x, [qt], bias)
    assert ops.last_kernel() in cluster_kernels
    assert out.dtype == act and within_one_ulp_16(out, want + bias.float().cpu().numpy()[None, :])


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("rows,k,m", [(5120, 17408, 1), (5120 + 7, 17408, 8), (3584, 18944, 4), (5120, 13824, 2)])
def test_large_matrices_of_few_rows_take_the_streaming_body_sliced_over_a_cluster(rows, k, m, bits):
    """Matrices of 16 MB and more that leave the tiled kernel about a CTA per SM or fewer: the
    streaming kernel's body, the reduction axis sliced over a thread-block cluster, the slices'
    sums added in slice order by the cluster's first CTA.  Against the oracle, with a bias, and the
    same bits on a second run."""
    from dynquant_b200 import ops

    meta = torch.float16 if (m + bits) % 2 else torch.bfloat16
    act = torch.float16 if m == 4 else torch.bfloat16
    qt = random_qt(rows, k, bits, meta=meta, seed=m * 10 + bits, offsets=bits != 4)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(act).cuda()
    bias = torch.randn(rows, generator=torch.Generator().manual_seed(7)).to(act).cuda()
    acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, 128, k, out_dtype=torch.float32)
    assert ops.last_kernel() == "gemv_mma_stream_sliced_kernel"
    want = oracle_gemv(x, qt)
    check_acc(acc, want)
    assert torch.equal(acc, ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, 128, k, out_dtype=torch.float32))
    out = ops.gemv_shards(x, [qt], bias)
    assert ops.last_kernel() == "gemv_mma_stream_sliced_kernel"
    assert out.dtype == act and within_one_ulp_16(out, want + bias.float().cpu().numpy()[None, :])


def test_many_rows_fused_shards_with_a_bias():
    from dynquant_b200 import _lib, ops

    m = 40
    x = torch.randn(m, 512, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    shards = [random_qt(12800, 512, 4, seed=1), random_qt(128, 512, 2, seed=2), random_qt(13000, 512, 8, seed=3)]
    bias = torch.randn(25928, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
    before = int(_lib.load().dq_launch_count())
    got = ops.gemv_row_chunks(x, shards, bias)
    # the two large shards two passes of twenty rows each; the small one as five chunks of eight rows in two launches
    assert int(_lib.load().dq_launch_count()) - before == 6
    want = torch.cat([ops.gemv_shards(x[i:i + 8].contiguous(), shards, bias) for i in range(0, m, 8)])
    assert got.shape == (m, 25928) and within_one_ulp_16(got, want.float().cpu().numpy())
    with pytest.raises(RuntimeError, match="exceeds the limit of 64"):
        ops.gemv_row_chunks(torch.zeros(65, 512, dtype=torch.bfloat16, device="cuda"), shards)


@pytest.mark.parametrize(("m", "launches"), [(9, 2), (16, 1), (20, 2), (32, 1), (33, 2), (64, 2)])
def test_row_chunks_share_launches(m, launches):
    """What the many-rows kernel does not take (here: a small matrix) runs as row chunks of equal
    size (+-1), up to four of them per launch of the tiled kernel (chunks of different sizes
    cannot share one), every row against the oracle."""
    from dynquant_b200 import _lib, ops

    qt = random_qt(1000, 1024, 3, seed=m)
    x = torch.randn(m, 1024, generator=torch.Generator().manual_seed(m)).to(torch.bfloat16).cuda()
    before = int(_lib.load().dq_launch_count())
    acc = ops.gemv_row_chunks(x, [qt], out_dtype=torch.float32)
    assert int(_lib.load().dq_launch_count()) - before == launches
    assert ops.last_kernel() == "gemv_mma_tile_kernel"
    check_acc(acc, oracle_gemv(x, qt))


def test_row_chunks_of_a_long_matrix_go_one_by_one():
    from dynquant_b200 import _lib, ops

    qt = random_qt(20480, 504, 4, seed=9)  # a padded last group: not the many-rows kernel's
    x = torch.randn(16, 504, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).cuda()
    before = int(_lib.load().dq_launch_count())
    acc = ops.gemv_row_chunks(x, [qt], out_dtype=torch.float32)
    assert int(_lib.load().dq_launch_count()) - before == 2 and ops.last_kernel().startswith("gemv_mma")
    check_acc(acc, oracle_gemv(x, qt))


@pytest.mark.parametrize(("widths", "m", "meta"), [
    ((4, 3), 1, torch.float16), ((2, 8), 1, torch.bfloat16), ((3, 8, 4), 8, torch.float16), ((2, 2, 4, 8), 3, torch.float16),
])
def test_long_fused_shards_take_the_streaming_body(widths, m, meta):
    """Two to four long matrices sharing an activation (a large model's gate / up): one launch,
    every matrix on its own range of CTAs running the streaming body of its width."""
    from dynquant_b200 import _lib, ops

    # >= 296 row tiles each and a tile per resident warp (3552) together; one row count ragged
    rows = {2: [28800, 28817], 3: [24000, 24017, 9600], 4: [19200, 19217, 9600, 9600]}[len(widths)]
    shards = [random_qt(r, 512, b, meta=meta, seed=10 * i + b) for i, (r, b) in enumerate(zip(rows, widths))]
    act = torch.bfloat16 if m != 3 else torch.float16
    x = torch.randn(m, 512, generator=torch.Generator().manual_seed(m)).to(act).cuda()
    before = int(_lib.load().dq_launch_count())
    acc = ops.gemv_shards(x, shards, out_dtype=torch.float32)
    assert int(_lib.load().dq_launch_count()) - before == 1
    assert ops.last_kernel() == "gemv_mma_stream_multi_kernel"
    col = 0
    got = acc.cpu().numpy()
    for s_, r in zip(shards, rows):
        want = oracle_gemv(x, s_)
        part = got[:, col:col + r]
        scale = np.abs(want).max() + 1e-30
        assert np.abs(part - want).max() / scale <= 1e-3, (s_.bits, r)
        col += r


# ---- (d) the head of the decode stack -----------------------------------------------------------


def test_the_248320_row_head():
    """248,320 x 2048 at 8 bits (45 % of the benchmark step's bytes): three slabs of its rows
    against the oracle, the rest through a row-sum identity -- the sum of all outputs equals the
    activation against the column sums of the dequantized matrix, here checked slab by slab on
    the GPU's own dequant (bit-exact elsewhere in this suite)."""
    from dynquant_b200 import ops

    rows, k = 248320, 2048
    qt = random_qt(rows, k, 8, seed=8)
    x = torch.randn(1, k, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).cuda()
    acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, 8, 128, k, out_dtype=torch.float32)
    assert ops.last_kernel() == "gemv_mma_stream_kernel"
    for lo, hi in ((0, 4096), (120000, 124096), (rows - 4099, rows)):
        check_acc(acc[:, lo:hi], oracle_gemv(x, qt.rows(lo, hi)))
    # every row, against dequant + matmul in double on the GPU
    total = 0.0
    worst = 0.0
    for lo in range(0, rows, 31040):
        part = qt.rows(lo, lo + 31040)
        dense = ops.dequant(part.packed, part.scales, part.offsets, 8, 128, k, out_dtype=torch.float32)
        ref = (dense.double() @ x.double().T).T
        worst = max(worst, float((acc[:, lo:lo + 31040].double() - ref).abs().max()))
        total = max(total, float(ref.abs().max()))
    assert worst / total <= 1e-3


# ---- (g) guarded output buffers -----------------------------------------------------------------

PAD = 64  # elements either side: 256 bytes of fp32


def guarded(m, rows, dtype):
    buf = torch.full((PAD + m * rows + PAD,), -12345.0, dtype=dtype, device="cuda")
    return buf, buf[PAD:PAD + m * rows].view(m, rows)


def guards_intact(buf, m, rows):
    return bool((buf[:PAD] == -12345.0).all()) and bool((buf[PAD + m * rows:] == -12345.0).all())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize(("rows", "k", "group"), GEOMETRIES + [(4097, 512, 128), (19001, 512, 128), (1000, 384, 128)])
def test_gemv_never_writes_outside_its_output(rows, k, group, bits, out_dtype):
    from dynquant_b200 import ops

    qt = make_quant(rows, k, group, bits, torch.float16).to("cuda") if rows < 4000 else random_qt(rows, k, bits, group)
    for m in (1, 5, 8):
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(torch.bfloat16).cuda()
        buf, out = guarded(m, rows, out_dtype)
        got = ops.gemv_shards(x, [qt], out_dtype=out_dtype, out=out)
        torch.cuda.synchronize()
        assert guards_intact(buf, m, rows), (ops.last_kernel(), m)
        assert not bool((got == -12345.0).any())  # and every element inside was written
        if out_dtype == torch.float32:
            check_acc(got, oracle_gemv(x, qt))


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize(("rows", "k", "group"), GEOMETRIES)
def test_dequant_never_writes_outside_its_output(rows, k, group, bits):
    from dynquant_b200 import _lib
    from dynquant_b200.ops import _stream, _tag, weight_descriptor

    qt = make_quant(rows, k, group, bits, torch.float16).to("cuda")
    buf, out = guarded(rows, k, torch.float16)
    w = weight_descriptor("dequant", qt.packed, qt.scales, qt.offsets, bits, qt.geometry.effective_group, k)
    _lib.check(_lib.load().dq_dequant(ctypes.byref(w), out.data_ptr(), _tag(torch.float16, "out"), _stream(out.device)))
    torch.cuda.synchronize()
    assert guards_intact(buf, rows, k)
    assert (out.cpu().view(torch.int16).numpy().view(np.uint16) == oracle_dequant(qt)).all()


def test_fused_shards_never_write_outside_their_output():
    from dynquant_b200 import ops

    k = 1024
    shards = [make_quant(rows, k, 128, bits, torch.float16, seed=60 + bits).to("cuda")
              for bits, rows in ((2, 96), (3, 161), (4, 33), (8, 7))]
    total = sum(q.num_rows for q in shards)
    for m in (1, 8):
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(torch.bfloat16).cuda()
        buf, out = guarded(m, total, torch.float32)
        got = ops.gemv_shards(x, shards, out_dtype=torch.float32, out=out)
        torch.cuda.synchronize()
        assert guards_intact(buf, m, total)
        check_acc(got, np.concatenate([oracle_gemv(x, q) for q in shards], axis=1))


# ---- (h) the two SIMT paths against each other --------------------------------------------------


@pytest.mark.parametrize("bits", BITS)
def test_the_two_simt_paths_agree(tmp_path, bits):
    """fp32 activations take the SIMT kernels: the chunked fast path here, the general
    block-at-a-time kernel in a child process started with DYNQUANT_GEMV_SCALAR=1 (the switch is
    read once per process, like the reference's).  Same integers, same scales, another summation
    order: they must agree to accumulation noise (2e-3, the reference's bar)."""
    from dynquant_b200 import ops

    saved = tmp_path / "general.pt"
    body = textwrap.dedent(
        f"""
        import sys
        sys.path.insert(0, {str(ROOT)!r})
        sys.path.insert(0, {str(ROOT / "tests")!r})
        import torch
        from conftest import make_quant
        from dynquant_b200 import ops
        qt = make_quant(260, 2048, 128, {bits}, torch.float32, seed=7).to("cuda")
        x = torch.randn(4, 2048, generator=torch.Generator().manual_seed(11)).cuda()
        y = ops.gemv(x, qt.packed, qt.scales, qt.offsets, {bits}, 128, 2048)
        WHICH
        torch.save(y.cpu(), {str(saved)!r})
        """
    )
    subprocess.run([sys.executable, "-c", body.replace("WHICH", 'assert ops.last_kernel() == "gemv_general_kernel"')],
                   check=True, env={**os.environ, "DYNQUANT_GEMV_SCALAR": "1"})
    qt = make_quant(260, 2048, 128, bits, torch.float32, seed=7).to("cuda")
    x = torch.randn(4, 2048, generator=torch.Generator().manual_seed(11)).cuda()
    fast = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, 128, 2048)
    assert ops.last_kernel() == "gemv_fast_kernel"
    general = torch.load(saved).cuda()
    torch.testing.assert_close(fast, general, rtol=2e-3, atol=2e-3)
    # and the tensor-core path on the same integers, with the activation rounded to bf16 first
    xb = x.to(torch.bfloat16)
    qh = make_quant(260, 2048, 128, bits, torch.float16, seed=7).to("cuda")
    mma = ops.gemv(xb, qh.packed, qh.scales, qh.offsets, bits, 128, 2048, out_dtype=torch.float32)
    assert ops.last_kernel().startswith("gemv_mma")
    check_acc(mma, oracle_gemv(xb, qh))


# ---- the reference's own CUDA kernel on the same inputs ------------------------------------------


@pytest.mark.parametrize("bits", BITS)
def test_agrees_with_the_references_own_cuda_gemv(tmp_path, bits):
    """``oracle/_ref/libdynquant_ref_cuda.so`` is the reference's gemv.cu / dequant.cu compiled
    where they lie (oracle/build_ref.py).  It runs in a child process (it registers the same
    operator namespace) on a tensor saved to disk; both outputs are bf16, compared at the
    reference's own bar for that dtype (rtol = atol = 2e-2, tests/test_kernels_parity.py:198-203),
    and the dequantized weights bit for bit."""
    lib = ROOT / "oracle" / "_ref" / "libdynquant_ref_cuda.so"
    if not lib.exists():
        pytest.skip("the reference's CUDA kernels are not built here")
    from dynquant_b200 import ops

    qt = make_quant(260, 2048, 128, bits, torch.bfloat16, seed=77)
    x = torch.randn(4, 2048, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
    torch.save({"packed": qt.packed, "scales": qt.scales, "offsets": qt.offsets, "x": x}, tmp_path / "in.pt")
    body = textwrap.dedent(
        f"""
        import torch
        torch.ops.load_library({str(lib)!r})
        d = torch.load({str(tmp_path / "in.pt")!r})
        args = [d[k].cuda() for k in ("packed", "scales", "offsets")]
        y = torch.ops.dynquant.gemv(d["x"].cuda(), *args, {bits}, 128, 2048)
        w = torch.ops.dynquant.dequant(*args, {bits}, 128, 2048)
        torch.save({{"y": y.cpu(), "w": w.cpu()}}, {str(tmp_path / "out.pt")!r})
        """
    )
    subprocess.run([sys.executable, "-c", body], check=True)
    ref = torch.load(tmp_path / "out.pt")
    dev = qt.to("cuda")
    got = ops.gemv(x.cuda(), dev.packed, dev.scales, dev.offsets, bits, 128, 2048)
    torch.testing.assert_close(got.float().cpu(), ref["y"].float(), rtol=2e-2, atol=2e-2)
    dense = ops.dequant(dev.packed, dev.scales, dev.offsets, bits, 128, 2048)
    assert torch.equal(dense.cpu().view(torch.int16), ref["w"].view(torch.int16))
