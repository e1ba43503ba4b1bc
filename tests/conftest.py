"""Shared test plumbing.

`-m "not gpu"` runs everything that needs no device (oracle, format, host logic,
C-ABI symbol checks, gloo multi-process tests); `-m gpu` runs the parity tests
proper, which call the CUDA kernels through the C ABI and compare with the CPU
oracle under ``oracle/``.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


TAG = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}


def raw(t: torch.Tensor | None) -> np.ndarray | None:
    """torch tensor -> the numpy array the oracle takes (16-bit floats as uint16 bit patterns)."""
    if t is None:
        return None
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.int32:
        return t.numpy().view(np.uint32)
    return t.numpy()


def from_raw(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    if dtype in (torch.float16, torch.bfloat16):
        return torch.from_numpy(a.view(np.int16).copy()).view(dtype)
    return torch.from_numpy(np.ascontiguousarray(a))


def make_quant(rows: int, in_features: int, group_size: int, bits: int, dtype: torch.dtype, *,
               seed: int | None = None, with_offsets: bool = True):
    """Seeded random packed tensor in the style of the reference's parity suite
    (tests/test_kernels_parity.py:72-92: manual_seed(bits*1000 + in_features), N(0,1) weights)."""
    from dynquant_b200 import QuantTensor

    gen = torch.Generator().manual_seed(bits * 1000 + in_features if seed is None else seed)
    dense = torch.randn(rows, in_features, generator=gen, dtype=torch.float32)
    qt = QuantTensor.from_dense(dense, bits=bits, group_size=group_size, compute_dtype=dtype)
    if not with_offsets:
        qt.offsets = None
    return qt


_VLLM_STATE = {"stack": None}


def vllm_world_of_one():
    """Once per process: a vLLM config context and a one-rank gloo world, which is all vLLM's
    parameter base class needs in order to construct (it reads the tensor-parallel rank off the
    process group).  The context stays open for the rest of the process."""
    import contextlib

    if _VLLM_STATE["stack"] is None:
        from vllm.config import DeviceConfig, VllmConfig, set_current_vllm_config
        from vllm.distributed import init_distributed_environment, initialize_model_parallel

        # (an explicit device: without a GPU vLLM cannot infer one, and none is needed for placement)
        device = "cuda" if torch.cuda.is_available() else "cpu"
        stack = contextlib.ExitStack()
        stack.enter_context(set_current_vllm_config(VllmConfig(device_config=DeviceConfig(device=device))))
        init_distributed_environment(world_size=1, rank=0, distributed_init_method="tcp://127.0.0.1:29541",
                                     local_rank=0, backend="gloo")
        initialize_model_parallel(1, 1)
        _VLLM_STATE["stack"] = stack
