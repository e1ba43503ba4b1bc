"""CPU oracle for the packed decode path -- TEST INFRASTRUCTURE, NOT PRODUCT.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module.  The shipped package (``dynquant_b200``) never does, and
has no CPU fallback.

Two independent restatements of the reference algorithm live here:

* ``np_*`` functions: vectorised numpy, written from the format specification
  (reference ``docs/format-spec.md:216-240`` for the word layout,
  ``docs/format-spec.md:124-134`` for ``w = q*scale + offset``) and following
  ``QuantTensor.dequantize`` (reference
  ``packages/dynquant-core/src/dynquant/quant/tensor.py:400-426``).
* ``c_*`` functions: ctypes bindings of ``dq_oracle.c`` (scalar C, follows the
  reference's ``dequant_cpu_rows`` / ``gemv_cpu``,
  ``packages/dynquant-kernels/csrc/bindings.cpp:84-117`` and ``:166-180``).

Arrays are numpy.  16-bit floats travel as ``uint16`` bit patterns together
with a dtype tag (``"f16"``, ``"bf16"``, ``"f32"``), because numpy has no
bfloat16.

Parity status: pinned.  ``tests/test_oracle.py`` checks both restatements
against the format specification's known-answer words, against golden vectors
generated from the reference's own Python implementation
(``tests/golden/make_golden.py``) and, where built, against the reference's
compiled CPU operators (``oracle/build_ref.py``).
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libdq_oracle.so"

DTYPE_TAGS = {"f16": 0, "bf16": 1, "f32": 2}
BITS = (2, 3, 4, 8)


# --------------------------------------------------------------------------
# geometry (reference: quant/pack.py:203-232 row_geometry)
# --------------------------------------------------------------------------


@dataclass(frozen=True)
class Geometry:
    bits: int
    group_values: int  # resolved count; == in_features when per-row
    num_groups: int
    words_per_group: int
    in_features: int
    per_row: bool

    @property
    def words_per_row(self) -> int:
        return self.num_groups * self.words_per_group

    @property
    def padded_in_features(self) -> int:
        return self.in_features if self.per_row else self.num_groups * self.group_values


def geometry(bits: int, group_size: int, in_features: int) -> Geometry:
    """``group_size == -1`` means one group spanning the row."""
    if bits not in BITS:
        raise ValueError(f"bits={bits} not supported")
    if in_features <= 0:
        raise ValueError("in_features must be positive")
    if group_size == -1:
        return Geometry(bits, in_features, 1, -(-in_features * bits // 32), in_features, True)
    if group_size <= 0 or group_size % 32:
        raise ValueError(f"group_size={group_size} must be a positive multiple of 32 (or -1)")
    groups = -(-in_features // group_size)
    return Geometry(bits, group_size, groups, group_size * bits // 32, in_features, False)


# --------------------------------------------------------------------------
# 16-bit float bit patterns
# --------------------------------------------------------------------------


def to_f32(a: np.ndarray, tag: str) -> np.ndarray:
    if tag == "f32":
        return np.asarray(a, dtype=np.float32)
    a = np.asarray(a, dtype=np.uint16)
    if tag == "f16":
        return a.view(np.float16).astype(np.float32)
    if tag == "bf16":
        return (a.astype(np.uint32) << np.uint32(16)).view(np.float32)
    raise ValueError(tag)


def from_f32(a: np.ndarray, tag: str) -> np.ndarray:
    """Round fp32 to the tagged dtype (nearest-even); 16-bit results as uint16."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if tag == "f32":
        return a
    if tag == "f16":
        return a.astype(np.float16).view(np.uint16)
    if tag == "bf16":
        bits = a.view(np.uint32)
        nan = (bits & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
        lsb = (bits >> np.uint32(16)) & np.uint32(1)
        rounded = ((bits + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)
        quiet = ((bits >> np.uint32(16)) | np.uint32(0x40)).astype(np.uint16)
        return np.where(nan, quiet, rounded)
    raise ValueError(tag)


# --------------------------------------------------------------------------
# numpy restatement
# --------------------------------------------------------------------------


def np_pack(codes: np.ndarray, bits: int) -> np.ndarray:
    """codes [..., n] (any int dtype, values < 2**bits) -> uint32 [..., ceil(n*bits/32)]."""
    codes = np.asarray(codes)
    n = codes.shape[-1]
    nwords = -(-n * bits // 32)
    q = codes.astype(np.uint64)
    if q.size and int(q.max()) >> bits:
        raise ValueError("code out of range")
    bit = np.arange(n, dtype=np.uint64) * np.uint64(bits)
    word = (bit >> np.uint64(5)).astype(np.int64)
    shift = bit & np.uint64(31)
    wide = q << shift  # up to 39 bits: low 32 stay, the rest spills into word+1
    out = np.zeros(codes.shape[:-1] + (nwords + 1,), dtype=np.uint64)
    flat_out = out.reshape(-1, nwords + 1)
    flat_wide = wide.reshape(-1, n)
    rows = np.arange(flat_out.shape[0])[:, None]
    # a sum is an OR here: every value owns a disjoint bit range of its word
    np.add.at(flat_out, (rows, word[None, :]), flat_wide & np.uint64(0xFFFFFFFF))
    np.add.at(flat_out, (rows, word[None, :] + 1), flat_wide >> np.uint64(32))
    return out[..., :nwords].astype(np.uint32)


def np_unpack(words: np.ndarray, bits: int, n: int) -> np.ndarray:
    """uint32 [..., nwords] -> uint8 codes [..., n]."""
    words = np.asarray(words).astype(np.uint32)
    w64 = np.concatenate(
        [words.astype(np.uint64), np.zeros(words.shape[:-1] + (1,), dtype=np.uint64)], axis=-1
    )
    bit = np.arange(n, dtype=np.uint64) * np.uint64(bits)
    word = (bit >> np.uint64(5)).astype(np.int64)
    shift = bit & np.uint64(31)
    both = w64[..., word] | (w64[..., word + 1] << np.uint64(32))
    return ((both >> shift) & np.uint64((1 << bits) - 1)).astype(np.uint8)


def np_dequant(
    packed: np.ndarray,
    scales: np.ndarray,
    offsets: np.ndarray | None,
    meta_tag: str,
    geom: Geometry,
    out_tag: str | None = None,
) -> np.ndarray:
    """Dense [rows, in_features] in ``out_tag`` (default: the metadata dtype)."""
    out_tag = out_tag or meta_tag
    rows = packed.shape[0]
    grouped = np.asarray(packed).astype(np.uint32).reshape(rows, geom.num_groups, geom.words_per_group)
    codes = np_unpack(grouped, geom.bits, geom.group_values).astype(np.float32)
    dense = codes * to_f32(scales, meta_tag)[..., None]
    if offsets is not None:
        dense = dense + to_f32(offsets, meta_tag)[..., None]
    dense = dense.reshape(rows, geom.num_groups * geom.group_values)[:, : geom.in_features]
    return from_f32(dense.astype(np.float32), out_tag)


def np_gemv(
    x: np.ndarray,
    x_tag: str,
    packed: np.ndarray,
    scales: np.ndarray,
    offsets: np.ndarray | None,
    meta_tag: str,
    geom: Geometry,
) -> np.ndarray:
    """fp32 [m, rows]: x.float() @ dequant(fp32).T, accumulated in float64."""
    w = np_dequant(packed, scales, offsets, meta_tag, geom, "f32").astype(np.float64)
    return (to_f32(x, x_tag).astype(np.float64) @ w.T).astype(np.float32)


def np_moe(
    x, x_tag, topk_ids, topk_w, gate_up, down, *, inter: int, num_experts: int, h_round: str = "f32"
) -> np.ndarray:
    """Composition oracle for the expert layer; banks are (packed, scales, offsets, tag, geom)."""
    xf = to_f32(x, x_tag).astype(np.float64)
    tokens, hidden = xf.shape
    y = np.zeros((tokens, hidden), dtype=np.float64)
    cache: dict[int, tuple[np.ndarray, np.ndarray]] = {}

    def expert(e: int):
        if e not in cache:
            p, s, o, tag, g = gate_up
            rows = slice(e * 2 * inter, (e + 1) * 2 * inter)
            wgu = np_dequant(p[rows], s[rows], None if o is None else o[rows], tag, g, "f32")
            p, s, o, tag, g = down
            rows = slice(e * hidden, (e + 1) * hidden)
            wd = np_dequant(p[rows], s[rows], None if o is None else o[rows], tag, g, "f32")
            cache[e] = (wgu.astype(np.float64), wd.astype(np.float64))
        return cache[e]

    for t in range(tokens):
        for k in range(topk_ids.shape[1]):
            e = int(topk_ids[t, k])
            if e < 0 or e >= num_experts:
                continue
            wgu, wd = expert(e)
            gu = (wgu @ xf[t]).astype(np.float32)
            g, u = gu[:inter], gu[inter:]
            h = (g / (np.float32(1) + np.exp(-g, dtype=np.float32))) * u
            if h_round != "f32":
                h = to_f32(from_f32(h, h_round), h_round)
            d = (wd @ h.astype(np.float64)).astype(np.float32)
            y[t] += float(topk_w[t, k]) * d.astype(np.float64)
    return y.astype(np.float32)


# --------------------------------------------------------------------------
# C restatement (ctypes)
# --------------------------------------------------------------------------

_lib = None


def build(force: bool = False) -> Path:
    """Compile ``dq_oracle.c`` with the Makefile beside it."""
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < (_HERE / "dq_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-s"], check=True)
    return _LIB_PATH


class _Bank(ctypes.Structure):
    _fields_ = [
        ("packed", ctypes.c_void_p),
        ("scales", ctypes.c_void_p),
        ("offsets", ctypes.c_void_p),
        ("meta_dtype", ctypes.c_int),
        ("num_groups", ctypes.c_int64),
        ("words_per_group", ctypes.c_int64),
        ("group_values", ctypes.c_int64),
        ("in_features", ctypes.c_int64),
        ("bits", ctypes.c_int),
    ]


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            if os.environ.get("DQ_ORACLE_NO_BUILD"):
                raise FileNotFoundError(f"{_LIB_PATH} missing; run `make -C oracle`")
            build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        for name in ("dqo_pack", "dqo_unpack", "dqo_dequant", "dqo_gemv", "dqo_moe"):
            getattr(_lib, name).restype = ctypes.c_int
    return _lib


def _ptr(a: np.ndarray | None):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def _meta(a, tag):
    return _c(a, np.float32 if tag == "f32" else np.uint16)


def c_pack(codes: np.ndarray, bits: int) -> np.ndarray:
    codes = _c(codes, np.uint8)
    rows = int(np.prod(codes.shape[:-1], dtype=np.int64))
    n = codes.shape[-1]
    out = np.empty(codes.shape[:-1] + (-(-n * bits // 32),), dtype=np.uint32)
    rc = lib().dqo_pack(_ptr(codes), ctypes.c_int64(rows), ctypes.c_int64(n), bits, _ptr(out))
    if rc:
        raise ValueError(f"dqo_pack failed ({rc})")
    return out


def c_unpack(words: np.ndarray, bits: int, n: int) -> np.ndarray:
    words = _c(words, np.uint32)
    rows = int(np.prod(words.shape[:-1], dtype=np.int64))
    out = np.empty(words.shape[:-1] + (n,), dtype=np.uint8)
    rc = lib().dqo_unpack(_ptr(words), ctypes.c_int64(rows), ctypes.c_int64(n), bits, _ptr(out))
    if rc:
        raise ValueError(f"dqo_unpack failed ({rc})")
    return out


def c_dequant(packed, scales, offsets, meta_tag, geom: Geometry, out_tag: str | None = None):
    out_tag = out_tag or meta_tag
    packed = _c(packed, np.uint32)
    scales = _meta(scales, meta_tag)
    offsets = None if offsets is None else _meta(offsets, meta_tag)
    rows = packed.shape[0]
    out = np.empty((rows, geom.in_features), dtype=np.float32 if out_tag == "f32" else np.uint16)
    rc = lib().dqo_dequant(
        _ptr(packed), _ptr(scales), _ptr(offsets), DTYPE_TAGS[meta_tag],
        ctypes.c_int64(rows), ctypes.c_int64(geom.num_groups), ctypes.c_int64(geom.words_per_group),
        ctypes.c_int64(geom.group_values), ctypes.c_int64(geom.in_features), geom.bits,
        _ptr(out), DTYPE_TAGS[out_tag],
    )
    if rc:
        raise ValueError(f"dqo_dequant failed ({rc})")
    return out


def c_gemv(x, x_tag, packed, scales, offsets, meta_tag, geom: Geometry) -> np.ndarray:
    x = _meta(x, x_tag)
    packed = _c(packed, np.uint32)
    scales = _meta(scales, meta_tag)
    offsets = None if offsets is None else _meta(offsets, meta_tag)
    m, rows = x.shape[0], packed.shape[0]
    y = np.empty((m, rows), dtype=np.float32)
    rc = lib().dqo_gemv(
        _ptr(x), DTYPE_TAGS[x_tag], ctypes.c_int64(m), _ptr(packed), _ptr(scales), _ptr(offsets),
        DTYPE_TAGS[meta_tag], ctypes.c_int64(rows), ctypes.c_int64(geom.num_groups),
        ctypes.c_int64(geom.words_per_group), ctypes.c_int64(geom.group_values),
        ctypes.c_int64(geom.in_features), geom.bits, _ptr(y),
    )
    if rc:
        raise ValueError(f"dqo_gemv failed ({rc})")
    return y


def _bank(packed, scales, offsets, tag, geom: Geometry):
    keep = (_c(packed, np.uint32), _meta(scales, tag), None if offsets is None else _meta(offsets, tag))
    b = _Bank(
        _ptr(keep[0]), _ptr(keep[1]), _ptr(keep[2]), DTYPE_TAGS[tag], geom.num_groups,
        geom.words_per_group, geom.group_values, geom.in_features, geom.bits,
    )
    return b, keep


def c_moe(x, x_tag, topk_ids, topk_w, gate_up, down, *, inter: int, num_experts: int, h_round: str = "f32"):
    x = _meta(x, x_tag)
    tokens, hidden = x.shape
    ids = _c(topk_ids, np.int32)
    w = _c(topk_w, np.float32)
    gu, keep1 = _bank(*gate_up)
    dn, keep2 = _bank(*down)
    y = np.empty((tokens, hidden), dtype=np.float32)
    rc = lib().dqo_moe(
        _ptr(x), DTYPE_TAGS[x_tag], ctypes.c_int64(tokens), ctypes.c_int64(hidden),
        ctypes.c_int64(inter), _ptr(ids), _ptr(w), ctypes.c_int64(ids.shape[1]),
        ctypes.c_int64(num_experts), ctypes.byref(gu), ctypes.byref(dn), DTYPE_TAGS[h_round], _ptr(y),
    )
    del keep1, keep2
    if rc:
        raise ValueError(f"dqo_moe failed ({rc})")
    return y
