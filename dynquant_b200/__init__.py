"""dynquant_b200: the packed mixed-precision decode path of DynQuant for NVIDIA B200.

Only sm_100a CUDA kernels behind a C ABI (``include/dynquant_b200.h``); no CPU
path, no alternative backends.  Importing the package registers
``torch.ops.dynquant.*`` with the reference's operator schemas; the compiled
library itself is loaded on first use and its absence is an error, never a
silent fallback.
"""

from . import ops
from .format import (
    BIT_OPTIONS,
    DEFAULT_GROUP_SIZE,
    PER_ROW_GROUP_SIZE,
    PackingError,
    QuantTensor,
    RowGeometry,
    pack_nbit,
    row_geometry,
    unpack_nbit,
)
from .checkpoint import PackedCheckpoint, load_packed_checkpoint, save_packed_checkpoint
from .ops import dequantize, embedding_lookup, gemv_max_rows, quantized_matmul

ABI_VERSION = 2

ops.register_torch_ops()


def is_available() -> bool:
    """True when the compiled library loads and a CUDA device is visible."""
    import torch

    from . import _lib

    try:
        _lib.load()
    except _lib.LibraryUnavailableError:
        return False
    return torch.cuda.is_available()


def install_kernel_shim() -> str:
    """Make the reference runtime (``dynquant.runtime``) find THESE kernels: put the stand-in for
    its ``dynquant_kernels`` package (``dynquant_b200/shim``) first on ``sys.path``.  Call it
    before ``dynquant.runtime`` resolves its backend.  Returns the directory added."""
    import sys
    from pathlib import Path

    shim = str(Path(__file__).resolve().parent / "shim")
    if shim not in sys.path:
        sys.path.insert(0, shim)
    return shim


__all__ = [
    "ABI_VERSION",
    "BIT_OPTIONS",
    "DEFAULT_GROUP_SIZE",
    "PER_ROW_GROUP_SIZE",
    "PackedCheckpoint",
    "PackingError",
    "QuantTensor",
    "RowGeometry",
    "dequantize",
    "embedding_lookup",
    "gemv_max_rows",
    "install_kernel_shim",
    "is_available",
    "load_packed_checkpoint",
    "ops",
    "pack_nbit",
    "quantized_matmul",
    "row_geometry",
    "save_packed_checkpoint",
    "unpack_nbit",
]
