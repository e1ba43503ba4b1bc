"""The C-ABI shared library: it loads, exports every symbol the header declares, answers the
metadata calls and validates geometry on the host -- all without a GPU."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from dynquant_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "dynquant_b200.h").read_text()


def declared_symbols() -> list[str]:
    return sorted(set(re.findall(r"DQ_API\s+[\w\s\*]+?\b(dq_\w+)\s*\(", HEADER)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    names = declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/dynquant_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures and the header disagree"


def test_header_names_every_kernel_the_library_reports():
    """dq_last_kernel()'s documentation lists the names a caller can see; every name the sources
    pass to note_kernel() must be in that list (a new kernel is not silently undocumented)."""
    csrc = ROOT / "dynquant_b200" / "csrc"
    reported = set()
    for path in list(csrc.glob("*.cu")) + list(csrc.glob("*.cuh")):
        reported |= set(re.findall(r'note_kernel\("(\w+)"\)', path.read_text()))
    assert len(reported) >= 8
    doc = HEADER[HEADER.index("Name of the kernel the calling thread"):HEADER.index("dq_last_kernel(void)")]
    missing = sorted(name for name in reported if f'"{name}"' not in doc)
    assert not missing, f"kernel names missing from the dq_last_kernel documentation: {missing}"


def test_abi_constants_match_the_reference_numbers():
    lib = _lib.load()
    assert lib.dq_abi_version() == 2  # csrc/include/dynquant/abi.h:23
    assert lib.dq_gemv_max_rows() == 8  # abi.h:39
    assert lib.dq_built_with_cuda() == 1
    assert lib.dq_compiled_architectures() == b"sm_100a"
    for name, value in (("DQ_ABI_VERSION", 2), ("DQ_GROUP_SIZE_ALIGNMENT", 32), ("DQ_GEMV_MAX_ROWS", 8)):
        assert re.search(rf"#define {name} {value}\b", HEADER)


def _weight(rows=4, wpr=16, groups=1, gv=128, k=128, bits=4, meta=0):
    return _lib.Weight(16, 16, None, rows, wpr, groups, gv, k, bits, meta)


def _resolve(w):
    geo = _lib.Geometry()
    rc = _lib.load().dq_resolve_geometry(b"dequant", ctypes.byref(w), ctypes.byref(geo))
    return rc, geo, _lib.last_error()


def test_geometry_resolves_like_the_reference():
    rc, geo, _ = _resolve(_weight(rows=4, wpr=32, groups=2, gv=128, k=200, bits=4))
    assert rc == 0
    assert (geo.words_per_group, geo.blocks_per_group, geo.blocks_per_row, geo.in_features) == (16, 16, 32, 200)
    rc, geo, _ = _resolve(_weight(rows=7, wpr=1, groups=1, gv=4, k=4, bits=3))  # per-row conv1d
    assert rc == 0 and geo.blocks_per_group == 1


@pytest.mark.parametrize(
    "kwargs,fragment",
    [
        (dict(bits=5), "unsupported bit width"),
        (dict(gv=-1), "resolved positive count"),
        (dict(k=0), "in_features must be positive"),
        (dict(wpr=17, groups=2, gv=64, k=128), "not divisible"),
        (dict(wpr=8, groups=1, gv=128, k=128), "needs 16 words"),
        (dict(wpr=32, groups=2, gv=128, k=300), "short of in_features"),
        (dict(wpr=16, groups=1, gv=128, k=100), "single group must span the row"),
        (dict(wpr=10, groups=2, gv=36, k=72, bits=4), "multiple of 32"),
    ],
)
def test_geometry_errors_keep_the_reference_wording(kwargs, fragment):
    rc, _, msg = _resolve(_weight(**kwargs))
    assert rc == _lib.DQ_ERR_INVALID
    assert fragment in msg


def test_gemv_row_limit_is_checked_before_any_device_work():
    lib = _lib.load()
    w = _weight()
    rc = lib.dq_gemv(ctypes.c_void_p(16), 0, 9, ctypes.byref(w), ctypes.c_void_p(16), 0, None)
    assert rc == _lib.DQ_ERR_INVALID and "exceeds the kernel's limit" in _lib.last_error()


def test_torch_ops_are_registered_with_reference_schemas_and_have_fakes():
    import torch

    import dynquant_b200  # noqa: F401

    assert str(torch.ops.dynquant.gemv.default._schema) == (
        "dynquant::gemv(Tensor x, Tensor packed, Tensor scales, Tensor? offsets, int bits, "
        "int group_values, int in_features) -> Tensor"
    )
    assert str(torch.ops.dynquant.dequant.default._schema) == (
        "dynquant::dequant(Tensor packed, Tensor scales, Tensor? offsets, int bits, int group_values, "
        "int in_features) -> Tensor"
    )
    assert int(torch.ops.dynquant.abi_version()) == 2
    # fake (meta) implementations: shape and dtype inference without data
    packed = torch.empty(8, 16, dtype=torch.int32, device="meta")
    scales = torch.empty(8, 1, dtype=torch.float16, device="meta")
    x = torch.empty(3, 128, dtype=torch.float16, device="meta")
    y = torch.ops.dynquant.gemv(x, packed, scales, None, 4, 128, 128)
    assert y.shape == (3, 8) and y.dtype == torch.float16
    d = torch.ops.dynquant.dequant(packed, scales, None, 4, 128, 128)
    assert d.shape == (8, 128) and d.dtype == torch.float16


def test_there_is_no_cpu_fallback():
    import torch

    from dynquant_b200 import ops
    from dynquant_b200.format import QuantTensor

    qt = QuantTensor.from_dense(torch.randn(8, 128), bits=4)
    x = torch.randn(1, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU"):
        ops.gemv(x, qt.packed, qt.scales, qt.offsets, 4, 128, 128)
    with pytest.raises(RuntimeError):
        torch.ops.dynquant.gemv(x, qt.packed, qt.scales, qt.offsets, 4, 128, 128)
    with pytest.raises(RuntimeError, match="no CPU"):
        ops.quantized_matmul(x, qt)
