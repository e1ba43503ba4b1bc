"""Stand-in for the reference's ``dynquant_kernels`` package, backed by ``dynquant_b200``.

The reference runtime finds its compiled operators through a package of this name
(``packages/dynquant-core/src/dynquant/runtime/backend.py:96-161``): it reads ``ABI_VERSION``
without loading anything, asks ``is_available()``, and on success calls
``torch.ops.dynquant.{gemv, dequant, gemv_max_rows}`` (``runtime/ops.py:163-260``).  Putting
THIS directory ahead of the reference's own kernel package on ``sys.path``
(``dynquant_b200.install_kernel_shim()``) makes ``dynquant.runtime`` -- ``quantized_matmul``,
``DynQuantLinear``, the serving plugins -- run unchanged on the sm_100a kernels.

Same surface as ``packages/dynquant-kernels/src/dynquant_kernels/__init__.py:32-120``:
``ABI_VERSION``, ``__version__``, ``is_available()``, ``load_result()``, ``report()``.
Importing it never raises; a missing library or GPU shows up as ``is_available() == False``
with the reason in ``load_result()``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

ABI_VERSION: int = 2  # packages/dynquant-kernels/csrc/include/dynquant/abi.h:23
__version__ = "0.0+b200"


@dataclass(frozen=True)
class KernelLoadResult:
    ok: bool
    error: str = ""
    remedy: str = ""


_RESULT: KernelLoadResult | None = None


def load_result() -> KernelLoadResult:
    """Load the sm_100a library and register the operators; cached, never raises."""
    global _RESULT
    if _RESULT is None:
        try:
            import torch

            import dynquant_b200
            from dynquant_b200 import _lib

            lib = _lib.load()
            if int(lib.dq_abi_version()) != ABI_VERSION:
                _RESULT = KernelLoadResult(False, f"library reports ABI {lib.dq_abi_version()}, this shell is {ABI_VERSION}",
                                           "rebuild with `python -m dynquant_b200.build`")
            elif not torch.cuda.is_available():
                _RESULT = KernelLoadResult(False, "no CUDA device is visible", "the library has sm_100a kernels only")
            elif not dynquant_b200.is_available():
                _RESULT = KernelLoadResult(False, "dynquant_b200 reports itself unavailable",
                                           "python -m dynquant_b200.build")
            elif not hasattr(torch.ops.dynquant, "gemv"):
                _RESULT = KernelLoadResult(False, "torch.ops.dynquant.gemv is not registered",
                                           "another extension owns the dynquant namespace in this process")
            else:
                _RESULT = KernelLoadResult(True)
        except Exception as exc:  # noqa: BLE001 - detection must not raise
            _RESULT = KernelLoadResult(False, f"{type(exc).__name__}: {exc}", "python -m dynquant_b200.build")
    return _RESULT


def is_available() -> bool:
    return load_result().ok


def report() -> dict[str, Any]:
    res = load_result()
    out: dict[str, Any] = {"package": "dynquant_b200", "abi_version": ABI_VERSION, "available": res.ok}
    if res.ok:
        import torch

        out["compiled_architectures"] = torch.ops.dynquant.compiled_architectures()
        out["gemv_max_rows"] = int(torch.ops.dynquant.gemv_max_rows())
    else:
        out["error"], out["remedy"] = res.error, res.remedy
    return out
