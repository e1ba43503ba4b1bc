"""Seeded random shapes through every GEMV entry point against the oracle.

The fixed-shape tests pin the corners that were thought of; this one draws (rows, reduction
length, width, group size, activation rows, dtypes, offsets) from the ranges the kernels split
on -- short / tiled / streaming row counts with ragged tails, reduction axes of one to 148
steps (with many and with few factors of two), 64- and 128-value groups, per-row groups, odd
lengths that only the general kernel takes
-- and checks fp32 accumulators within 1e-3 of the oracle (the reference's own definition,
``tests/test_kernels_parity.py:198-199``: ``x.float() @ dequant(fp32).T``).  It also records
which kernel every case took and requires that the draw reached all of them, so a dispatch
change cannot silently leave a kernel outside this test.
"""

from __future__ import annotations

import random

import numpy as np
import pytest
import torch

from conftest import make_quant
from test_gpu_parity import oracle_gemv
from test_gpu_shapes import random_qt

pytestmark = pytest.mark.gpu

PER_ROW = -1


def _draw(rng: random.Random):
    kind = rng.choice(["short", "tiled", "tiled", "stream", "rows_x_long_k", "few_factors", "general"])
    bits = rng.choice([2, 3, 4, 8])
    x_dtype = rng.choice([torch.bfloat16, torch.float16])
    meta = rng.choice([torch.float16, torch.bfloat16])
    offsets = rng.random() < 0.8
    m = rng.choice([1, 1, 2, 3, 5, 8])
    group = 128
    if kind == "short":
        rows, k = rng.randint(1, 300), 128 * rng.randint(1, 12)
        group = rng.choice([64, 128])
    elif kind == "tiled":
        rows, k = rng.randint(301, 9000), 128 * rng.choice([2, 4, 6, 8, 16, 32])
        group = rng.choice([64, 128, 128])
    elif kind == "stream":
        rows, k = rng.randint(18944, 36000), 512 * rng.choice([1, 2, 4])
    elif kind == "rows_x_long_k":
        rows, k, m = rng.randint(16, 700), 128 * rng.choice([56, 96, 112]), rng.choice([4, 8, 8])
    elif kind == "few_factors":  # step counts the tiled kernel slices badly, few rows: the many-rows kernel, sliced over a cluster
        rows, k = rng.randint(1300, 4200), 128 * rng.choice([70, 86, 148, 74, 106])
        group = rng.choice([64, 128])
    else:  # lengths and groups only the SIMT kernels take
        rows = rng.randint(1, 200)
        k, group = rng.choice([(100, PER_ROW), (320, 32), (4304, 128), (72, PER_ROW), (2048 + 64, 64)])
        x_dtype = rng.choice([torch.bfloat16, torch.float16, torch.float32])
    return kind, rows, k, bits, group, m, x_dtype, meta, offsets


def test_random_shapes_match_the_oracle_and_reach_every_kernel():
    from dynquant_b200 import ops

    rng = random.Random(20261)
    seen: dict[str, int] = {}
    for case in range(160):
        kind, rows, k, bits, group, m, x_dtype, meta, offsets = _draw(rng)
        if kind in ("stream", "few_factors"):  # (generated on the device: encoding 70 M values on the host takes seconds)
            qt = random_qt(rows, k, bits, group=group, meta=meta, seed=case, offsets=offsets)
        else:
            qt = make_quant(rows, k, group, bits, meta, seed=case, with_offsets=offsets).to("cuda")
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(case)).to(x_dtype).cuda()
        acc = ops.gemv(x, qt.packed, qt.scales, qt.offsets, bits, qt.geometry.effective_group, k, out_dtype=torch.float32)
        name = ops.last_kernel()
        seen[name] = seen.get(name, 0) + 1
        want = oracle_gemv(x, qt)
        got = acc.cpu().numpy()
        scale = np.abs(want).max() + 1e-30
        err = float(np.abs(got - want).max() / scale)
        assert err <= 1e-3, (case, kind, rows, k, bits, group, m, x_dtype, meta, offsets, name, err)
        assert np.linalg.norm(got - want) / (np.linalg.norm(want) + 1e-30) <= 1e-3, (case, kind, name)
    for kernel in ("gemv_mma_tile_kernel", "gemv_mma_stream_kernel", "gemv_rows_kernel", "gemv_fast_kernel", "gemv_general_kernel"):
        assert seen.get(kernel, 0) >= 3, (kernel, seen)
    assert seen.get("gemv_mma_stream_sliced_kernel", 0) >= 1, seen  # (few of the draws are matrices of 16 MB and more)


def test_random_fused_shards_and_row_chunks_match_the_oracle():
    """Fused layers of two to four shards of mixed widths, 1..40 activation rows (chunks above
    eight), a bias on some: every shard's columns against the oracle."""
    from dynquant_b200 import ops

    rng = random.Random(977)
    for case in range(40):
        k = 128 * rng.choice([2, 4, 8, 16, 32])
        meta = rng.choice([torch.float16, torch.bfloat16])
        shards = [make_quant(16 * rng.randint(1, 160) + rng.choice([0, 0, 5]), k, 128, rng.choice([2, 3, 4, 8]), meta,
                             seed=100 * case + i).to("cuda") for i in range(rng.randint(2, 4))]
        m = rng.choice([1, 2, 4, 8, 9, 16, 24, 40])
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(case)).to(torch.bfloat16).cuda()
        total = sum(s.num_rows for s in shards)
        bias = torch.randn(total, generator=torch.Generator().manual_seed(case)).cuda() if rng.random() < 0.4 else None
        fn = ops.gemv_shards if m <= 8 else ops.gemv_row_chunks
        got = fn(x, shards, bias, out_dtype=torch.float32).cpu().numpy()
        col = 0
        for s in shards:
            want = oracle_gemv(x, s)
            if bias is not None:
                want = want + bias[col:col + s.num_rows].cpu().numpy()[None, :]
            part = got[:, col:col + s.num_rows]
            scale = np.abs(want).max() + 1e-30
            assert np.abs(part - want).max() / scale <= 1e-3, (case, m, k, s.bits, s.num_rows)
            col += s.num_rows
