"""Path A: the REFERENCE's own Python runtime running on this library's operators.

``dynquant.runtime.ops.quantized_matmul`` / ``DynQuantLinear`` (reference
``packages/dynquant-core/src/dynquant/runtime/ops.py:184-231``, ``runtime/linear.py:174-212``)
are used unmodified; only the kernel package they probe for is replaced by the stand-in in
``dynquant_b200/shim``.  The reference's Python sources are not part of this repository: the
tests run where ``DYNQUANT_REFERENCE_SRC`` points at its ``packages/dynquant-core/src`` and are
skipped elsewhere.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

from conftest import make_quant

SRC = os.environ.get("DYNQUANT_REFERENCE_SRC", "")
needs_reference = pytest.mark.skipif(not (SRC and os.path.isdir(os.path.join(SRC, "dynquant"))),
                                     reason="DYNQUANT_REFERENCE_SRC does not point at the reference's Python sources")


def test_shim_has_the_surface_the_reference_probes():
    """backend.py:96-161 reads ABI_VERSION, __version__, is_available(), load_result(), report()."""
    import dynquant_b200

    shim = dynquant_b200.install_kernel_shim()
    assert sys.path[0] == shim
    import dynquant_kernels as K

    assert K.ABI_VERSION == 2 and isinstance(K.__version__, str)
    res = K.load_result()
    assert K.is_available() == res.ok
    rep = K.report()
    assert rep["abi_version"] == 2 and rep["available"] == res.ok
    if not torch.cuda.is_available():
        assert not res.ok and res.error and res.remedy  # the reason is reported, nothing raises


@needs_reference
@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_reference_runtime_runs_on_these_operators(bits):
    import dynquant_b200
    from test_gpu_parity import oracle_gemv

    dynquant_b200.install_kernel_shim()
    sys.path.insert(1, SRC)
    os.environ.pop("DYNQUANT_BACKEND", None)
    from dynquant.quant.tensor import QuantTensor as RefTensor
    from dynquant.runtime import ops as R
    from dynquant.runtime.linear import DynQuantLinear as RefLinear

    qt = make_quant(96, 1024, 128, bits, torch.float16).to("cuda")
    ref_qt = RefTensor(packed=qt.packed, scales=qt.scales, offsets=qt.offsets, bits=bits, group_size=128,
                       in_features=1024, logical_shape=(96, 1024))
    assert R.uses_compiled_kernels(ref_qt), "the reference runtime did not select its compiled-kernel backend"
    assert int(R.gemv_max_rows()) == 8
    for m in (1, 5, 20):  # GEMV, GEMV, and the reference's dequant + dense path above 8 rows
        x = torch.randn(m, 1024, generator=torch.Generator().manual_seed(m)).to(torch.float16).cuda()
        got = R.quantized_matmul(x, ref_qt)
        want = oracle_gemv(x, qt)
        torch.testing.assert_close(got.float().cpu(), torch.from_numpy(want), rtol=2e-2, atol=2e-2)
    dense = R.dequantize(ref_qt)
    assert torch.equal(dense, qt.dequantize())
    layer = RefLinear(ref_qt, torch.zeros(96, dtype=torch.float16, device="cuda"))
    x = torch.randn(2, 3, 1024, dtype=torch.float16, device="cuda")
    y = layer(x)
    assert y.shape == (2, 3, 96)
    torch.testing.assert_close(y.float().cpu().reshape(6, 96), torch.from_numpy(oracle_gemv(x.reshape(6, 1024), qt)),
                               rtol=2e-2, atol=2e-2)
