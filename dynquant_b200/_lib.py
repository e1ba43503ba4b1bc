"""ctypes binding of ``libdynquant_b200.so`` (the C ABI in ``include/dynquant_b200.h``).

There is deliberately no fallback: if the library is missing or a call fails,
an exception is raised.  Nothing in this package computes the packed GEMV on
the CPU or through another backend.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libdynquant_b200.so"

DQ_F16, DQ_BF16, DQ_F32 = 0, 1, 2
DQ_OK, DQ_ERR_INVALID, DQ_ERR_CUDA, DQ_ERR_UNSUPPORTED, DQ_ERR_DEVICE = 0, 1, 2, 3, 4


class LibraryUnavailableError(RuntimeError):
    """The compiled sm_100a library is not present or cannot be loaded."""


class Weight(ctypes.Structure):
    """``dq_weight``."""

    _fields_ = [
        ("packed", ctypes.c_void_p),
        ("scales", ctypes.c_void_p),
        ("offsets", ctypes.c_void_p),
        ("rows", ctypes.c_int64),
        ("words_per_row", ctypes.c_int64),
        ("num_groups", ctypes.c_int64),
        ("group_values", ctypes.c_int64),
        ("in_features", ctypes.c_int64),
        ("bits", ctypes.c_int32),
        ("meta_dtype", ctypes.c_int32),
    ]


class Geometry(ctypes.Structure):
    """``dq_geometry``."""

    _fields_ = [
        ("group_values", ctypes.c_int32),
        ("num_groups", ctypes.c_int32),
        ("words_per_group", ctypes.c_int32),
        ("words_per_row", ctypes.c_int32),
        ("in_features", ctypes.c_int32),
        ("blocks_per_group", ctypes.c_int32),
        ("blocks_per_row", ctypes.c_int32),
    ]


class GemvJob(ctypes.Structure):
    """``dq_gemv_job``."""

    _fields_ = [
        ("x", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("m", ctypes.c_int64),
        ("out_stride", ctypes.c_int64),
        ("out_col0", ctypes.c_int64),
        ("x_dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("weight", Weight),
    ]


class PlanInfo(ctypes.Structure):
    """``dq_plan_info``."""

    _fields_ = [
        ("num_stages", ctypes.c_int32),
        ("num_jobs", ctypes.c_int32),
        ("grid", ctypes.c_int32),
        ("threads", ctypes.c_int32),
        ("ring_slots", ctypes.c_int32),
        ("launches", ctypes.c_int32),
        ("shared_bytes", ctypes.c_int64),
    ]


class PeerGroup(ctypes.Structure):
    """``dq_peer_group``."""

    _fields_ = [
        ("buffers", ctypes.c_void_p),
        ("buffer_bytes", ctypes.c_int64),
        ("world", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("spin_limit", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
    ]


class PeerPush(ctypes.Structure):
    """``dq_peer_push``."""

    _fields_ = [
        ("windows", ctypes.POINTER(ctypes.c_void_p)),
        ("world", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("data_offset", ctypes.c_int64),
        ("piece_bytes", ctypes.c_int64),
        ("flags_offset", ctypes.c_int64),
        ("state_offset", ctypes.c_int64),
        ("status_offset", ctypes.c_int64),
        ("spin_limit", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
    ]


_P = ctypes.c_void_p
_I32 = ctypes.c_int32
_I64 = ctypes.c_int64
_WP = ctypes.POINTER(Weight)

# name -> (restype, argtypes); every symbol include/dynquant_b200.h declares.
SIGNATURES = {
    "dq_abi_version": (_I32, []),
    "dq_built_with_cuda": (_I32, []),
    "dq_compiled_architectures": (ctypes.c_char_p, []),
    "dq_gemv_max_rows": (_I32, []),
    "dq_launch_count": (_I64, []),
    "dq_last_kernel": (ctypes.c_char_p, []),
    "dq_moe_max_tokens": (_I32, []),
    "dq_last_error": (ctypes.c_char_p, []),
    "dq_resolve_geometry": (_I32, [ctypes.c_char_p, _WP, ctypes.POINTER(Geometry)]),
    "dq_dequant": (_I32, [_WP, _P, _I32, _P]),
    "dq_probe_read": (_I32, [_P, _I64, _P, _P]),
    "dq_probe_copy": (_I32, [_P, _P, _I64, _P]),
    "dq_gemv": (_I32, [_P, _I32, _I64, _WP, _P, _I32, _P]),
    "dq_gemv_shards": (_I32, [_P, _I32, _I64, _WP, _I32, _P, _P, _I64, _I32, _P]),
    "dq_gemv_shards_rows": (_I32, [_P, _I32, _I64, _WP, _I32, _P, _P, _I64, _I32, _P]),
    "dq_gemv_sequence": (_I32, [ctypes.POINTER(GemvJob), _I32, _P]),
    "dq_moe_scratch_bytes": (_I32, [_I64, _I64, _I64, _I64, _I64, _I32, ctypes.POINTER(ctypes.c_int64)]),
    "dq_moe_gemv": (_I32, [_P, _I32, _I64, _P, _P, _I64, _I64, _WP, _WP, _I64, _I64, _P, _I32, _P, _I64, _P]),
    "dq_moe_gemv_shard": (_I32, [_P, _I32, _I64, _P, _P, _I64, _I64, _I64, _WP, _WP, _I64, _I64, _P, _I32, _P, _I64, _P]),
    "dq_moe_gemv_static": (_I32, [_P, _I32, _I64, _P, _P, _I64, _I64, _WP, _WP, _I64, _I64, _P, _I32, _P]),
    "dq_plan_workspace_bytes": (_I32, [_I32, ctypes.POINTER(ctypes.c_int64)]),
    "dq_plan_create": (_I32, [ctypes.POINTER(GemvJob), _I32, _P, _I64, _P, ctypes.POINTER(_P)]),
    "dq_plan_launch": (_I32, [_P, _P]),
    "dq_plan_status": (_I32, [_P, _P]),
    "dq_plan_describe": (_I32, [_P, ctypes.POINTER(PlanInfo)]),
    "dq_plan_stage_shape": (_I32, [_P, _I32, ctypes.POINTER(_I32), ctypes.POINTER(_I32), ctypes.POINTER(_I32)]),
    "dq_plan_set_wait": (_I32, [_P, _I32, _I32, _I32, _P]),
    "dq_plan_destroy": (None, [_P]),
    "dq_peer_header_bytes": (_I64, []),
    "dq_peer_all_gather": (_I32, [ctypes.POINTER(PeerGroup), _P, _I64, _P, _P]),
    "dq_peer_reduce_scatter_f32": (_I32, [ctypes.POINTER(PeerGroup), _P, _I64, _P, _I32, _P]),
    "dq_peer_status": (_I32, [ctypes.POINTER(PeerGroup), _P, _P]),
    "dq_peer_all_gather_parts": (_I32, [ctypes.POINTER(PeerGroup), ctypes.POINTER(ctypes.c_void_p),
                                        ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_void_p), _I32, _P]),
    "dq_gemv_stage_push": (_I32, [ctypes.POINTER(GemvJob), _I32, ctypes.POINTER(PeerPush), _P]),
    "dq_peer_push_status": (_I32, [ctypes.POINTER(PeerPush), _P]),
    "dq_gemv_host": (_I32, [_P, _I32, _I64, _WP, _P, _I32, _P, _P, _P]),
}

_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise LibraryUnavailableError(
                f"{LIB_PATH} is missing. Build it with `python -m dynquant_b200.build` "
                "(needs nvcc; targets sm_100a). There is no CPU or alternative backend."
            )
        try:
            lib = ctypes.CDLL(str(LIB_PATH))
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise LibraryUnavailableError(f"cannot load {LIB_PATH}: {exc}") from exc
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                raise LibraryUnavailableError(f"{LIB_PATH} does not export {name}; rebuild it")
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def last_error() -> str:
    return load().dq_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raise like the reference's operators do: RuntimeError with its message."""
    if status != DQ_OK:
        raise RuntimeError(last_error() or f"dynquant_b200 call failed with status {status}")
