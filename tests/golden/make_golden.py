"""Generate the golden vectors in this folder from the REFERENCE implementation.

Run in a container where the reference checkout is mounted::

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py [--reference <checkout>]

It imports the reference's own Python package (``dynquant.quant.pack``,
``dynquant.quant.tensor``, ``dynquant.runtime.ops`` on the torch backend) and writes
``golden_v1.npz``: for a list of seeded small cases the packed words the reference's
``pack_nbit`` produces, the metadata its ``QuantTensor.from_dense`` derives, its
``QuantTensor.dequantize`` output (bit patterns), the fp32 test oracle
``x.float() @ dequantize(fp32).T`` of ``tests/test_kernels_parity.py:198-199`` and the
output of its torch path ``quantized_matmul``.  The vectors travel with the repository;
the reference does not.
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

# (rows, in_features, group_size, bits, meta dtype, activation rows, with offsets)
CASES = [
    (6, 512, 128, 2, "f16", 1, True),
    (5, 512, 128, 3, "f16", 2, True),
    (6, 512, 128, 4, "bf16", 3, True),
    (4, 512, 128, 8, "f16", 1, True),
    (5, 320, 128, 3, "f16", 2, True),      # pad tail
    (3, 320, 128, 4, "bf16", 1, False),    # no offsets
    (4, 128, 32, 2, "f16", 4, True),       # smallest group
    (4, 128, 32, 3, "f16", 1, True),
    (6, 100, -1, 3, "f16", 2, True),       # per-row, ragged tail
    (7, 4, -1, 3, "f16", 1, True),         # fewer values than a 3-bit block
    (7, 4, -1, 8, "f16", 1, True),
    (3, 256, 64, 4, "f32", 5, True),       # fp32 metadata
    (3, 1024, 128, 3, "bf16", 8, True),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ns = ap.parse_args()
    os.environ["DYNQUANT_BACKEND"] = "torch"
    sys.path.insert(0, str(Path(ns.reference) / "packages" / "dynquant-core" / "src"))
    import torch
    from dynquant.quant.pack import pack_nbit, unpack_nbit
    from dynquant.quant.tensor import QuantTensor
    from dynquant.runtime import ops as ref_ops

    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}

    def raw(t):
        t = t.contiguous()
        if t.dtype in (torch.float16, torch.bfloat16):
            return t.view(torch.int16).numpy().view(np.uint16).copy()
        if t.dtype == torch.int32:
            return t.numpy().view(np.uint32).copy()
        return t.numpy().copy()

    out = {}
    # format-spec known answer: q[i] = i mod 8 at 3-bit
    kat = pack_nbit(torch.arange(32) % 8, 3)
    out["kat3_words"] = raw(kat)
    # bijection at awkward sizes (reference tests/test_pack.py:28-37)
    for bits in (2, 3, 4, 8):
        for n in (1, 2, 3, 7, 8, 31, 32, 33, 37, 96, 127, 128, 129, 1023):
            g = torch.Generator().manual_seed(bits * 10000 + n)
            q = torch.randint(0, 1 << bits, (2, n), generator=g)
            words = pack_nbit(q, bits)
            assert torch.equal(unpack_nbit(words, bits, n).to(torch.int64), q)
            out[f"pack_b{bits}_n{n}_codes"] = q.to(torch.uint8).numpy()
            out[f"pack_b{bits}_n{n}_words"] = raw(words)

    for ci, (rows, k, group, bits, meta, m, with_off) in enumerate(CASES):
        torch.manual_seed(bits * 1000 + k)
        dense = torch.randn(rows, k)
        qt = QuantTensor.from_dense(dense, bits=bits, group_size=group, compute_dtype=dt[meta])
        if not with_off:
            qt.offsets = None
        torch.manual_seed(m)
        x = torch.randn(m, k).to(torch.bfloat16 if meta == "bf16" else torch.float16)
        key = f"case{ci}"
        out[f"{key}_spec"] = np.array([rows, k, group, bits, m, int(with_off)], dtype=np.int64)
        out[f"{key}_meta"] = np.array(meta)
        out[f"{key}_dense"] = dense.numpy()
        out[f"{key}_packed"] = raw(qt.packed)
        out[f"{key}_scales"] = raw(qt.scales)
        if with_off:
            out[f"{key}_offsets"] = raw(qt.offsets)
        out[f"{key}_dequant"] = raw(qt.dequantize())
        out[f"{key}_dequant_f32"] = raw(qt.dequantize(dtype=torch.float32))
        out[f"{key}_x"] = raw(x)
        out[f"{key}_x_tag"] = np.array("bf16" if x.dtype == torch.bfloat16 else "f16")
        out[f"{key}_y32"] = (x.float() @ qt.dequantize(dtype=torch.float32).T).numpy()
        out[f"{key}_y_torch_path"] = raw(ref_ops.quantized_matmul(x, qt))
    np.savez_compressed(HERE / "golden_v1.npz", **out)
    print(f"wrote {HERE / 'golden_v1.npz'} with {len(out)} arrays")


if __name__ == "__main__":
    main()
