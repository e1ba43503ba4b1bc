"""Compile the CUDA sources into ``dynquant_b200/lib/libdynquant_b200.so``.

sm_100a only.  Invoked by ``python -m dynquant_b200.build`` and by the repo's
build entry point; needs ``nvcc`` but no GPU (it cross-compiles).  The library
has no dependency on torch or Python: it is the C ABI of ``include/dynquant_b200.h``.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
OBJ_DIR = PKG / "lib" / "obj"
LIB_PATH = PKG / "lib" / "libdynquant_b200.so"

SOURCES = ["dq_capi.cu", "dq_dequant.cu", "dq_gemv.cu", "dq_gemv_mma.cu", "dq_gemv_plan.cu", "dq_gemv_rows.cu", "dq_gemv_stream_multi.cu", "dq_gemv_stream_sliced.cu", "dq_moe.cu", "dq_peer.cu", "dq_probe.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "-I", str(INCLUDE), "-I", str(CSRC),
]


def nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(path).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build dynquant_b200")
    return path


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False, tuning: bool = False) -> Path:
    """``tuning``: compile in the launch-shape overrides (``DQ_B200_*`` environment variables read
    at every launch) that the sweeps behind the built-in heuristics used; not for normal use."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    # The objects remember which kind of build they are: switching between the normal and the
    # tuning build recompiles everything (time stamps alone would keep the other kind's objects).
    stamp = OBJ_DIR / "build_kind.txt"
    kind = "tuning" if tuning else "normal"
    if not stamp.exists() or stamp.read_text().strip() != kind:
        force = True
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h")) + [Path(__file__)]
    sources = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc(), *NVCC_FLAGS, *(["-DDQ_TUNING"] if tuning else []), "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd: list[str]) -> None:
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0 or ptxas_info:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {cmd[-3]}")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(run, jobs))
    stamp.write_text(kind + "\n")
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    if jobs or force or _stale(LIB_PATH, objs):
        run([nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs),
             "-Xlinker", "-rpath,/usr/local/cuda/lib64"])
    return LIB_PATH


TORCH_SHIM_PATH = PKG / "lib" / "libdynquant_b200_torch.so"


def build_torch_shim(force: bool = False, verbose: bool = False) -> Path | None:
    """Compile ``csrc/dq_torch_shim.cpp`` -- the C++ CUDA backend of ``torch.ops.dynquant.{gemv,
    dequant}`` -- against the installed torch and link it to the C-ABI library beside it.  It is
    optional: without it the operators are implemented by a Python function over ctypes (same
    kernels, more host time per call).  Returns None when no C++ compiler is available."""
    src = CSRC / "dq_torch_shim.cpp"
    if not force and not _stale(TORCH_SHIM_PATH, [src, INCLUDE / "dynquant_b200.h", LIB_PATH]):
        return TORCH_SHIM_PATH
    gxx = shutil.which("g++")
    if gxx is None or not LIB_PATH.exists():
        return None
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = [gxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I", str(INCLUDE), "-I", sysconfig.get_paths()["include"], "-I", "/usr/local/cuda/include"]
    for p in cpp_extension.include_paths():
        cmd += ["-isystem", p]
    cmd += [str(src), "-o", str(TORCH_SHIM_PATH), "-L", str(LIB_PATH.parent), "-ldynquant_b200",
            "-L", str(torch_lib), "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("g++ failed on dq_torch_shim.cpp")
    return TORCH_SHIM_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv or "--tuning" in sys.argv, verbose=True,
                         ptxas_info="--ptxas-info" in sys.argv, tuning="--tuning" in sys.argv)
    print(path)
    print(build_torch_shim(force="--force" in sys.argv, verbose=True))
