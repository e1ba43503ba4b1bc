"""Compile the REFERENCE's own C++ CPU operators into ``oracle/_ref/`` -- test infrastructure.

The reference ships CPU implementations of ``dynquant::dequant`` and
``dynquant::gemv`` in one self-contained source file
(``packages/dynquant-kernels/csrc/bindings.cpp:84-180``, headers under
``packages/dynquant-kernels/csrc/include``).  This script compiles that file
*where it lies* in the reference checkout, with g++ against the installed torch
headers, and writes only ``oracle/_ref/libdynquant_ref_cpu.so``.  No reference
source is copied into this repository, and the reference's own build system
(CMake / scikit-build) is not run.

The result is used (a) to validate the C and numpy restatements in this folder
and (b) as the timed CPU baseline (``kind: "reference"``).  It needs the
reference checkout only at build time; the built library travels.

    python oracle/build_ref.py [--reference /path/to/checkout]
"""

from __future__ import annotations

import argparse
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
OUT = OUT_DIR / "libdynquant_ref_cpu.so"
DEFAULT_REFERENCE = Path("/root/reference")


def build(reference: Path = DEFAULT_REFERENCE, force: bool = False) -> Path | None:
    """Returns the library path, or None when the reference checkout is absent."""
    src = reference / "packages" / "dynquant-kernels" / "csrc" / "bindings.cpp"
    inc = reference / "packages" / "dynquant-kernels" / "csrc" / "include"
    if not src.exists():
        return OUT if OUT.exists() else None
    if OUT.exists() and not force and OUT.stat().st_mtime >= src.stat().st_mtime:
        return OUT
    import torch
    from torch.utils import cpp_extension

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I", str(inc), "-I", sysconfig.get_paths()["include"]]
    for p in cpp_extension.include_paths():
        cmd += ["-isystem", p]
    cmd += [str(src), "-o", str(OUT), "-L", str(torch_lib), "-ltorch", "-ltorch_cpu", "-lc10",
            f"-Wl,-rpath,{torch_lib}"]
    subprocess.run(cmd, check=True)
    return OUT


OUT_CUDA = OUT_DIR / "libdynquant_ref_cuda.so"


def build_cuda(reference: Path = DEFAULT_REFERENCE, force: bool = False) -> Path | None:
    """The reference's own CUDA GEMV and dequant (``csrc/gemv/gemv.cu``, ``csrc/quant/dequant.cu``)
    plus its operator schemas (``csrc/bindings.cpp``), compiled where they lie with nvcc for the
    architecture its CMake would pick on this toolkit (``100-real``,
    ``packages/dynquant-kernels/CMakeLists.txt:153-165``) into ``oracle/_ref/libdynquant_ref_cuda.so``.
    It is the second baseline of the sweep -- the reference's SIMT kernels on the same B200 -- and
    is only ever loaded by a child process of a benchmark or test.  Returns None when the
    checkout or nvcc is missing."""
    import shutil

    csrc = reference / "packages" / "dynquant-kernels" / "csrc"
    sources = [csrc / "bindings.cpp", csrc / "gemv" / "gemv.cu", csrc / "quant" / "dequant.cu"]
    if not all(p.exists() for p in sources):
        return OUT_CUDA if OUT_CUDA.exists() else None
    if OUT_CUDA.exists() and not force and OUT_CUDA.stat().st_mtime >= max(p.stat().st_mtime for p in sources):
        return OUT_CUDA
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        return None
    import torch
    from torch.utils import cpp_extension

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = [nvcc, "-O3", "-std=c++17", "-shared", "-x", "cu", "--expt-relaxed-constexpr",
           "-gencode", "arch=compute_100,code=sm_100",
           "-Xcompiler", "-fPIC,-fvisibility=hidden",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I", str(csrc / "include"), "-I", sysconfig.get_paths()["include"]]
    for p in cpp_extension.include_paths():
        cmd += ["-isystem", p]
    cmd += [str(p) for p in sources]
    cmd += ["-o", str(OUT_CUDA), "-L", str(torch_lib), "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-Xlinker", f"-rpath,{torch_lib}"]
    subprocess.run(cmd, check=True)
    return OUT_CUDA


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    ns = ap.parse_args()
    path = build(ns.reference, ns.force)
    print(path if path else "reference checkout not found; nothing built")
    path = build_cuda(ns.reference, ns.force)
    print(path if path else "reference CUDA kernels not built (no checkout or no nvcc)")
    sys.exit(0)
