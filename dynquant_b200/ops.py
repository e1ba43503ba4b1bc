"""Operators over packed tensors, backed by the sm_100a library only.

Two layers:

* plain functions (``gemv``, ``dequant``, ``gemv_shards``, ...) taking torch
  CUDA tensors and calling the C ABI with raw pointers on torch's current
  stream;
* the dispatcher operators ``torch.ops.dynquant.{gemv, dequant, abi_version,
  built_with_cuda, compiled_architectures, gemv_max_rows}`` registered with the
  same schema strings as the reference extension
  (``packages/dynquant-kernels/csrc/bindings.cpp:184-215``) plus fake (meta)
  implementations like ``packages/dynquant-kernels/src/dynquant_kernels/ops.py:81-122``,
  so code written against ``torch.ops.dynquant.*`` runs unchanged.  If another
  extension already owns the ``dynquant`` namespace in this process the
  registration is skipped and the plain functions remain available.

And the dispatch layer of the reference runtime
(``packages/dynquant-core/src/dynquant/runtime/ops.py:163-260``):
``dequantize``, ``quantized_matmul`` and ``embedding_lookup`` with the same
signatures and the same rule -- at most ``gemv_max_rows()`` activation rows go
to the packed GEMV, more go to dequant + a dense matmul.  There is no torch or
CPU fallback here: a tensor that is not on a CUDA device raises.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import DQ_BF16, DQ_F16, DQ_F32, Weight
from .format import QuantTensor

_DTYPE_TAG = {torch.float16: DQ_F16, torch.bfloat16: DQ_BF16, torch.float32: DQ_F32}


def _tag(dtype: torch.dtype, what: str) -> int:
    try:
        return _DTYPE_TAG[dtype]
    except KeyError:
        raise RuntimeError(f"{what}: unsupported dtype {dtype}; expected float16, bfloat16 or float32") from None


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"{what} is on {t.device}; dynquant_b200 has only sm_100a kernels and no CPU fallback"
        )


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def weight_descriptor(
    op: str,
    packed: torch.Tensor,
    scales: torch.Tensor,
    offsets: torch.Tensor | None,
    bits: int,
    group_values: int,
    in_features: int,
) -> Weight:
    """Shape/dtype checks an ``at::Tensor`` signature implies, then the POD the C ABI takes.

    Mirrors the tensor-level half of ``resolve_geometry``
    (``csrc/include/dynquant/geometry.h:71-86``); the arithmetic half runs in C.
    """
    if packed.dim() != 2:
        raise RuntimeError(f"{op}: packed must be 2-D [rows, words], got {tuple(packed.shape)}")
    if packed.dtype != torch.int32:
        raise RuntimeError(
            f"{op}: packed must be int32 (unsigned bit patterns stored as int32), got {packed.dtype}"
        )
    if scales.dim() != 2:
        raise RuntimeError(f"{op}: scales must be 2-D [rows, groups], got {tuple(scales.shape)}")
    if packed.shape[0] != scales.shape[0]:
        raise RuntimeError(f"{op}: packed has {packed.shape[0]} rows but scales has {scales.shape[0]}")
    if not (packed.is_contiguous() and scales.is_contiguous()):
        raise RuntimeError(f"{op}: packed and scales must be contiguous")
    _require_cuda(packed, f"{op}: packed")
    if scales.device != packed.device:
        raise RuntimeError(f"{op}: scales is on {scales.device} but packed is on {packed.device}")
    if offsets is not None:
        if offsets.shape != scales.shape:
            raise RuntimeError(f"{op}: offsets shape {tuple(offsets.shape)} != scales shape {tuple(scales.shape)}")
        if offsets.dtype != scales.dtype:
            raise RuntimeError(f"{op}: offsets dtype {offsets.dtype} != scales dtype {scales.dtype}")
        if not offsets.is_contiguous():
            raise RuntimeError(f"{op}: offsets must be contiguous")
        if offsets.device != packed.device:
            raise RuntimeError(f"{op}: offsets is on {offsets.device} but packed is on {packed.device}")
    return Weight(
        packed.data_ptr(),
        scales.data_ptr(),
        None if offsets is None else offsets.data_ptr(),
        packed.shape[0],
        packed.shape[1],
        scales.shape[1],
        int(group_values),
        int(in_features),
        int(bits),
        _tag(scales.dtype, f"{op}: scales"),
    )


# --------------------------------------------------------------------------
# plain functions
# --------------------------------------------------------------------------


def dequant(
    packed: torch.Tensor,
    scales: torch.Tensor,
    offsets: torch.Tensor | None,
    bits: int,
    group_values: int,
    in_features: int,
    *,
    out_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """Dense ``[rows, in_features]`` in the scales dtype (or ``out_dtype``)."""
    lib = _lib.load()
    w = weight_descriptor("dequant", packed, scales, offsets, bits, group_values, in_features)
    geom = _lib.Geometry()
    _lib.check(lib.dq_resolve_geometry(b"dequant", ctypes.byref(w), ctypes.byref(geom)))
    out_dtype = out_dtype or scales.dtype
    out = torch.empty((packed.shape[0], in_features), dtype=out_dtype, device=packed.device)
    if out.numel() == 0:
        return out
    with torch.cuda.device(packed.device):
        _lib.check(lib.dq_dequant(ctypes.byref(w), out.data_ptr(), _tag(out_dtype, "dequant: out"), _stream(packed.device)))
    return out


def _check_x(op: str, x: torch.Tensor, packed: torch.Tensor, in_features: int) -> None:
    if x.dim() != 2:
        raise RuntimeError(f"{op}: x must be 2-D [rows, in_features], got {tuple(x.shape)}")
    if x.shape[1] != in_features:
        raise RuntimeError(f"{op}: x has {x.shape[1]} columns but in_features is {in_features}")
    if not x.is_contiguous():
        raise RuntimeError(f"{op}: x must be contiguous")
    _require_cuda(x, f"{op}: x")
    if x.device != packed.device:
        raise RuntimeError(f"{op}: x is on {x.device} but the weight is on {packed.device}")


def gemv(
    x: torch.Tensor,
    packed: torch.Tensor,
    scales: torch.Tensor,
    offsets: torch.Tensor | None,
    bits: int,
    group_values: int,
    in_features: int,
    *,
    out_dtype: torch.dtype | None = None,
    strict_dtypes: bool = False,
) -> torch.Tensor:
    """``x @ W.T`` with ``W`` packed; ``x`` is ``[M <= 8, in_features]``.

    ``out_dtype`` defaults to ``x.dtype`` (the reference's behaviour);
    ``torch.float32`` returns the unrounded accumulators.  Unlike the reference
    operator (``csrc/gemv/gemv.cu:706-707``) the activation dtype may differ
    from the scales dtype unless ``strict_dtypes`` is set.
    """
    lib = _lib.load()
    w = weight_descriptor("gemv", packed, scales, offsets, bits, group_values, in_features)
    geom = _lib.Geometry()
    _lib.check(lib.dq_resolve_geometry(b"gemv", ctypes.byref(w), ctypes.byref(geom)))
    _check_x("gemv", x, packed, in_features)
    if strict_dtypes and x.dtype != scales.dtype:
        raise RuntimeError(f"gemv: x dtype {x.dtype} != scales dtype {scales.dtype}")
    out_dtype = out_dtype or x.dtype
    m = x.shape[0]
    out = torch.empty((m, packed.shape[0]), dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(
            lib.dq_gemv(
                x.data_ptr(), _tag(x.dtype, "gemv: x"), m, ctypes.byref(w), out.data_ptr(),
                _tag(out_dtype, "gemv: out"), _stream(x.device),
            )
        )
    return out


# Up to this many activation rows a packed matmul is issued as GEMV launches of
# ``gemv_max_rows()`` rows each: re-reading the packed weights (mostly from L2) a few times
# is cheaper than writing the dense weight out and reading it back, which is what the
# dequantize + dense path costs.  Measured on B200 for a 14336 x 4096 layer at 16 rows:
# two GEMV launches ~45 us against ~215-275 us for dequantize + matmul.
GEMV_CHUNKED_MAX_ROWS = 64


def gemv_row_chunks(
    x: torch.Tensor,
    shards: list[QuantTensor],
    bias: torch.Tensor | None = None,
    *,
    out_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """``gemv_shards`` for more rows than one launch takes, up to ``GEMV_CHUNKED_MAX_ROWS``: the
    library cuts the rows into chunks of at most ``gemv_max_rows()`` and issues up to four
    (chunk, shard) pairs per launch (``dq_gemv_shards_rows``)."""
    return gemv_shards(x, shards, bias, out_dtype=out_dtype, _entry="dq_gemv_shards_rows")


def gemv_shards(
    x: torch.Tensor,
    shards: list[QuantTensor],
    bias: torch.Tensor | None = None,
    *,
    out_dtype: torch.dtype | None = None,
    out: torch.Tensor | None = None,
    _entry: str = "dq_gemv_shards",
) -> torch.Tensor:
    """All shards of a fused layer against one activation; outputs concatenated along the last dim.

    ``out`` (optional): a contiguous ``[m, total_rows]`` tensor to write into instead of a new one."""
    lib = _lib.load()
    if not shards:
        raise RuntimeError("gemv_shards: need at least one shard")
    in_features = shards[0].in_features
    arr = (Weight * len(shards))()
    for i, qt in enumerate(shards):
        arr[i] = weight_descriptor(
            "gemv_shards", qt.packed, qt.scales, qt.offsets, qt.bits, qt.geometry.effective_group, qt.in_features
        )
    _check_x("gemv_shards", x, shards[0].packed, in_features)
    out_dtype = out_dtype or x.dtype
    total = sum(qt.num_rows for qt in shards)
    if bias is not None:
        if bias.shape != (total,) or bias.dtype != out_dtype or not bias.is_contiguous():
            raise RuntimeError(f"gemv_shards: bias must be a contiguous [{total}] tensor of {out_dtype}")
    m = x.shape[0]
    if out is None:
        out = torch.empty((m, total), dtype=out_dtype, device=x.device)
    elif out.shape != (m, total) or out.dtype != out_dtype or not out.is_contiguous() or out.device != x.device:
        raise RuntimeError(f"gemv_shards: out must be a contiguous [{m}, {total}] {out_dtype} tensor on {x.device}")
    with torch.cuda.device(x.device):
        _lib.check(
            getattr(lib, _entry)(
                x.data_ptr(), _tag(x.dtype, "gemv_shards: x"), m, arr, len(shards),
                None if bias is None else bias.data_ptr(), out.data_ptr(), total,
                _tag(out_dtype, "gemv_shards: out"), _stream(x.device),
            )
        )
    return out


def gemv_host(
    x_host: torch.Tensor,
    qt: QuantTensor,
    out_host: torch.Tensor,
    x_dev: torch.Tensor,
    out_dev: torch.Tensor,
) -> torch.Tensor:
    """The C ABI's host-buffer entry point: copy in, launch, copy out, synchronise."""
    lib = _lib.load()
    w = weight_descriptor("gemv", qt.packed, qt.scales, qt.offsets, qt.bits, qt.geometry.effective_group, qt.in_features)
    if x_host.is_cuda or out_host.is_cuda:
        raise RuntimeError("gemv_host: x_host and out_host must be host tensors")
    m = x_host.shape[0]
    with torch.cuda.device(qt.device):
        _lib.check(
            lib.dq_gemv_host(
                x_host.data_ptr(), _tag(x_host.dtype, "gemv_host: x"), m, ctypes.byref(w),
                out_host.data_ptr(), _tag(out_host.dtype, "gemv_host: out"),
                x_dev.data_ptr(), out_dev.data_ptr(), _stream(qt.device),
            )
        )
    return out_host


def moe_scratch_bytes(tokens: int, topk: int, hidden: int, inter: int, num_experts: int, act_dtype: torch.dtype) -> int:
    n = ctypes.c_int64(0)
    _lib.check(_lib.load().dq_moe_scratch_bytes(tokens, topk, hidden, inter, num_experts, _tag(act_dtype, "moe"), ctypes.byref(n)))
    return int(n.value)


def moe_gemv(
    x: torch.Tensor,
    topk_ids: torch.Tensor,
    topk_weights: torch.Tensor,
    gate_up: QuantTensor,
    down: QuantTensor,
    *,
    num_experts: int,
    out_dtype: torch.dtype | None = None,
    scratch: torch.Tensor | None = None,
    first_expert: int = 0,
) -> torch.Tensor:
    """Expert layer over packed banks: ``sum_k w[t,k] * down_e(silu(gate_e(x_t)) * up_e(x_t))``.

    ``first_expert``: the banks hold experts ``[first_expert, first_expert + num_experts)`` of a
    larger layer and ``topk_ids`` carry the layer's global numbers (one rank of an
    expert-parallel layer); ids outside that range are skipped.

    ``gate_up`` is the bank ``[E, 2*inter, hidden]`` folded to rows (gate rows of an expert
    first), ``down`` is ``[E, hidden, inter]`` folded to rows; ``topk_ids`` int32
    ``[tokens, topk]`` with ids outside ``[0, num_experts)`` skipped; ``topk_weights`` fp32.
    ``scratch`` (uint8, CUDA) may be passed to avoid an allocation per call.
    """
    lib = _lib.load()
    if x.dim() != 2 or not x.is_contiguous():
        raise RuntimeError(f"moe_gemv: x must be a contiguous 2-D [tokens, hidden] tensor, got {tuple(x.shape)}")
    _require_cuda(x, "moe_gemv: x")
    tokens, hidden = x.shape
    inter = down.in_features
    if topk_ids.dtype != torch.int32 or topk_ids.dim() != 2 or topk_ids.shape[0] != tokens or not topk_ids.is_contiguous():
        raise RuntimeError("moe_gemv: topk_ids must be a contiguous int32 [tokens, topk] tensor")
    if topk_weights.dtype != torch.float32 or topk_weights.shape != topk_ids.shape or not topk_weights.is_contiguous():
        raise RuntimeError("moe_gemv: topk_weights must be a contiguous float32 tensor shaped like topk_ids")
    topk = topk_ids.shape[1]
    wgu = weight_descriptor("moe_gemv", gate_up.packed, gate_up.scales, gate_up.offsets, gate_up.bits,
                            gate_up.geometry.effective_group, gate_up.in_features)
    wdn = weight_descriptor("moe_gemv", down.packed, down.scales, down.offsets, down.bits,
                            down.geometry.effective_group, down.in_features)
    out_dtype = out_dtype or x.dtype
    need = moe_scratch_bytes(tokens, topk, hidden, inter, num_experts, x.dtype)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    elif scratch.numel() < need or scratch.dtype != torch.uint8 or scratch.device != x.device:
        raise RuntimeError(f"moe_gemv: scratch must be a uint8 tensor of at least {need} bytes on {x.device}")
    y = torch.empty((tokens, hidden), dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(
            lib.dq_moe_gemv_shard(
                x.data_ptr(), _tag(x.dtype, "moe_gemv: x"), tokens, topk_ids.data_ptr(), topk_weights.data_ptr(),
                topk, first_expert, num_experts, ctypes.byref(wgu), ctypes.byref(wdn), hidden, inter, y.data_ptr(),
                _tag(out_dtype, "moe_gemv: out"), scratch.data_ptr(), scratch.numel(), _stream(x.device),
            )
        )
    return y


def moe_max_tokens() -> int:
    return int(_lib.load().dq_moe_max_tokens())


def gemv_max_rows() -> int:
    return int(_lib.load().dq_gemv_max_rows())


def launch_count() -> int:
    """Kernels the library has launched in this process so far (``dq_launch_count``)."""
    return int(_lib.load().dq_launch_count())


def last_kernel() -> str:
    """Name of the kernel this thread's last GEMV call launched (``dq_last_kernel``)."""
    return _lib.load().dq_last_kernel().decode()


def probe_read(buf: torch.Tensor, sink: torch.Tensor) -> None:
    """One read-only pass over ``buf`` (``dq_probe_read``); XOR of its 32-bit words into ``sink[0]``."""
    _require_cuda(buf, "probe_read: buffer")
    if not buf.is_contiguous() or sink.dtype != torch.int64 or sink.device != buf.device:
        raise RuntimeError("probe_read: expected a contiguous buffer and an int64 sink on the same device")
    nbytes = buf.numel() * buf.element_size()
    with torch.cuda.device(buf.device):
        _lib.check(_lib.load().dq_probe_read(buf.data_ptr(), nbytes, sink.data_ptr(), _stream(buf.device)))


def probe_copy(dst: torch.Tensor, src: torch.Tensor) -> None:
    """``dst <- src`` through the library's streaming copy kernel (``dq_probe_copy``)."""
    _require_cuda(src, "probe_copy: source")
    _require_cuda(dst, "probe_copy: destination")
    nbytes = src.numel() * src.element_size()
    if not (src.is_contiguous() and dst.is_contiguous()) or dst.numel() * dst.element_size() != nbytes:
        raise RuntimeError("probe_copy: expected two contiguous buffers of the same size in bytes")
    if dst.device != src.device:
        raise RuntimeError("probe_copy: both buffers must be on one device")
    with torch.cuda.device(src.device):
        _lib.check(_lib.load().dq_probe_copy(dst.data_ptr(), src.data_ptr(), nbytes, _stream(src.device)))


def achievable_bandwidth(nbytes: int = 4 << 30, iters: int = 10, device: torch.device | None = None) -> dict:
    """Read and copy bandwidth this GPU delivers right now, in GB/s, timed with CUDA events.

    The reference measures the same pair with ``src.sum()`` and ``dst.copy_(src)`` on 1 GiB
    (commands/bench.py:95-120); the default here is 4 GiB read and 2 GiB copied to 2 GiB so
    that a 126 MB L2 serves a negligible part.  The buffers are released before returning.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    nbytes = max(16, nbytes // 32 * 32)
    with torch.cuda.device(device):
        buf = torch.empty(nbytes // 8, dtype=torch.int64, device=device)
        buf.random_()
        sink = torch.zeros(1, dtype=torch.int64, device=device)
        half = buf.numel() // 2
        src, dst = buf[:half], buf[half:]

        def timed(fn) -> float:
            for _ in range(2):
                fn()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(device)
            start.record()
            for _ in range(iters):
                fn()
            stop.record()
            torch.cuda.synchronize(device)
            return start.elapsed_time(stop) * 1e-3 / iters

        read_s = timed(lambda: probe_read(buf, sink))
        copy_s = timed(lambda: probe_copy(dst, src))
        result = {
            "read_gbs": nbytes / read_s / 1e9,
            "copy_gbs": 2 * (nbytes // 2) / copy_s / 1e9,
            "bytes": nbytes,
            "iters": iters,
        }
        del buf, src, dst, sink
        torch.cuda.empty_cache()
    return result


# --------------------------------------------------------------------------
# runtime dispatch (reference: runtime/ops.py)
# --------------------------------------------------------------------------


def _kernel_args(qt: QuantTensor):
    """Positional arguments shared by ``dequant`` and ``gemv`` (``runtime/ops.py:146-160``)."""
    if qt.layout != "linear":
        raise NotImplementedError(
            f"the compiled kernels read linear layout; this tensor is {qt.layout}."
        )
    return (qt.packed, qt.scales, qt.offsets, qt.bits, qt.geometry.effective_group, qt.in_features)


def dequantize(qt: QuantTensor, *, dtype: torch.dtype | None = None) -> torch.Tensor:
    """Reconstruct the dense tensor (``runtime/ops.py:163-181``)."""
    dense = dequant(*_kernel_args(qt))
    dense = dense.reshape(qt.logical_shape)
    return dense if dtype is None else dense.to(dtype)


def quantized_matmul(x: torch.Tensor, qt: QuantTensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ W.T + bias`` where ``W`` is stored packed (``runtime/ops.py:184-231``)."""
    if x.shape[-1] != qt.in_features:
        raise ValueError(
            f"activation has {x.shape[-1]} input features but the weight expects {qt.in_features}"
        )
    if len(qt.logical_shape) != 2:
        raise ValueError(f"quantized_matmul expects a 2-D weight; this tensor is {qt.logical_shape}.")
    lead = x.shape[:-1]
    flat = x.reshape(-1, qt.in_features)
    if bias is not None and bias.dtype != flat.dtype:
        bias = bias.to(flat.dtype)
    args = _kernel_args(qt)
    if flat.shape[0] <= gemv_max_rows():
        if bias is None:
            # the operator's C++ backend when it is loaded: a third of the host time of the
            # Python route over ctypes (same entry point of the library underneath)
            out = torch.ops.dynquant.gemv(flat.contiguous(), *args) if _native_backend else gemv(flat.contiguous(), *args)
        else:
            out = gemv_shards(flat.contiguous(), [qt], bias.contiguous())
    elif flat.shape[0] <= GEMV_CHUNKED_MAX_ROWS and flat.is_cuda:
        out = gemv_row_chunks(flat.contiguous(), [qt], None if bias is None else bias.contiguous())
    else:
        weight = dequant(*args)
        out = torch.nn.functional.linear(flat, weight.to(x.dtype), bias)
    return out.reshape(*lead, qt.num_rows)


def embedding_lookup(qt: QuantTensor, ids: torch.Tensor) -> torch.Tensor:
    """Gather rows of a packed table, then dequantize only those (``runtime/ops.py:234-260``)."""
    if len(qt.logical_shape) != 2:
        raise ValueError(f"embedding table must be 2-D, got {qt.logical_shape}")
    flat_ids = ids.reshape(-1)
    packed, scales, offsets, bits, group_values, in_features = _kernel_args(qt)
    rows = packed.index_select(0, flat_ids)
    meta_scales = scales.index_select(0, flat_ids)
    meta_offsets = None if offsets is None else offsets.index_select(0, flat_ids)
    dense = dequant(rows, meta_scales, meta_offsets, bits, group_values, in_features)
    return dense.reshape(*ids.shape, in_features)


# --------------------------------------------------------------------------
# torch.ops.dynquant.* registration
# --------------------------------------------------------------------------

_registered = False
_libs: list[torch.library.Library] = []


_native_backend = False


def torch_ops_backend() -> str:
    """``"c++"`` when ``torch.ops.dynquant.{gemv,dequant}`` run through the compiled shim
    (``lib/libdynquant_b200_torch.so``, built by ``python -m dynquant_b200.build``), ``"python"``
    when they are Python functions over ctypes."""
    return "c++" if _native_backend else "python"


def _load_torch_shim() -> bool:
    import os
    from pathlib import Path

    if os.environ.get("DQ_B200_TORCH_SHIM", "1") == "0":
        return False
    path = Path(__file__).resolve().parent / "lib" / "libdynquant_b200_torch.so"
    if not path.exists():
        return False
    try:
        _lib.load()
        torch.ops.load_library(str(path))
    except (OSError, RuntimeError, _lib.LibraryUnavailableError):
        return False  # built against another torch, or the C-ABI library is missing: Python backend
    return True


def register_torch_ops() -> bool:
    """Define ``torch.ops.dynquant.*`` with the reference's schema strings.  Idempotent."""
    global _registered
    if _registered:
        return True
    try:
        lib = torch.library.Library("dynquant", "DEF")
    except RuntimeError:
        # Another extension already defined the namespace (e.g. the reference's own
        # CPU build loaded as the test oracle).  Leave it alone.
        return False
    lib.define("abi_version() -> int")
    lib.define("built_with_cuda() -> bool")
    lib.define("compiled_architectures() -> str")
    lib.define("gemv_max_rows() -> int")
    lib.define(
        "dequant(Tensor packed, Tensor scales, Tensor? offsets, int bits, int group_values, "
        "int in_features) -> Tensor"
    )
    lib.define(
        "gemv(Tensor x, Tensor packed, Tensor scales, Tensor? offsets, int bits, "
        "int group_values, int in_features) -> Tensor"
    )
    lib.impl("abi_version", lambda: int(_lib.load().dq_abi_version()), "CompositeExplicitAutograd")
    lib.impl("built_with_cuda", lambda: bool(_lib.load().dq_built_with_cuda()), "CompositeExplicitAutograd")
    lib.impl(
        "compiled_architectures",
        lambda: _lib.load().dq_compiled_architectures().decode(),
        "CompositeExplicitAutograd",
    )
    lib.impl("gemv_max_rows", lambda: int(_lib.load().dq_gemv_max_rows()), "CompositeExplicitAutograd")

    def _dequant_cuda(packed, scales, offsets, bits, group_values, in_features):
        return dequant(packed, scales, offsets, bits, group_values, in_features)

    def _gemv_cuda(x, packed, scales, offsets, bits, group_values, in_features):
        return gemv(x, packed, scales, offsets, bits, group_values, in_features)

    def _no_cpu(name):
        def raiser(*args, **kwargs):
            raise RuntimeError(
                f"dynquant::{name}: tensors are on the CPU; this build has only sm_100a kernels "
                "and deliberately no CPU implementation"
            )

        return raiser

    # CUDA backend: the compiled C++ shim when it has been built (one dispatcher hop and one C
    # call per operator call), else these Python functions over ctypes.  Same kernels either way.
    global _native_backend
    _native_backend = _load_torch_shim()
    if not _native_backend:
        lib.impl("dequant", _dequant_cuda, "CUDA")
        lib.impl("gemv", _gemv_cuda, "CUDA")
    lib.impl("dequant", _no_cpu("dequant"), "CPU")
    lib.impl("gemv", _no_cpu("gemv"), "CPU")

    @torch.library.register_fake("dynquant::dequant", lib=lib)
    def _dequant_fake(packed, scales, offsets, bits, group_values, in_features):
        torch._check(packed.dim() == 2, lambda: f"dequant: packed must be 2-D, got {tuple(packed.shape)}")
        torch._check(scales.dim() == 2, lambda: f"dequant: scales must be 2-D, got {tuple(scales.shape)}")
        torch._check(
            packed.shape[0] == scales.shape[0],
            lambda: f"dequant: {packed.shape[0]} packed rows vs {scales.shape[0]} scale rows",
        )
        return scales.new_empty((packed.shape[0], in_features))

    @torch.library.register_fake("dynquant::gemv", lib=lib)
    def _gemv_fake(x, packed, scales, offsets, bits, group_values, in_features):
        torch._check(x.dim() == 2, lambda: f"gemv: x must be 2-D, got {tuple(x.shape)}")
        torch._check(packed.dim() == 2, lambda: f"gemv: packed must be 2-D, got {tuple(packed.shape)}")
        torch._check(
            x.shape[1] == in_features,
            lambda: f"gemv: x has {x.shape[1]} columns but in_features is {in_features}",
        )
        return x.new_empty((x.shape[0], packed.shape[0]))

    _libs.append(lib)
    _registered = True
    return True
