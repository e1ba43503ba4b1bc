"""Time the reference's CPU path for the packed GEMV -- test/benchmark infrastructure.

Run as a child process by ``bench.py`` (its ``cpu_baseline`` leg and its
``--impl reference`` arm).  It must NOT import ``dynquant_b200``: when the
reference's compiled CPU operators are available (``oracle/_ref``, built by
``oracle/build_ref.py``) they register the ``dynquant::`` operator namespace
themselves.  Otherwise the C restatement ``dq_oracle.c`` is timed (``kind:
"port"``, one thread).

    python oracle/cpu_baseline.py '<json spec>'

spec = {"modules": [[rows, in_features, bits], ...], "m": 1, "repeat": 1, "seed": 7, "threads": 16}
("threads": host threads torch may use -- set explicitly so the figure does not depend on an
OMP_NUM_THREADS a launcher put into the environment)
prints {"kind", "cores", "seconds", "bytes", "gbps", "modules"} as one JSON line.
"""

from __future__ import annotations

import json
import os
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_LIB = HERE / "_ref" / "libdynquant_ref_cpu.so"


def main() -> None:
    spec = json.loads(sys.argv[1])
    import numpy as np
    import torch

    if spec.get("threads"):
        torch.set_num_threads(int(spec["threads"]))
    gen = torch.Generator().manual_seed(int(spec.get("seed", 7)))
    m = int(spec.get("m", 1))
    group = 128
    mods = []
    total_bytes = 0
    for rows, k, bits in spec["modules"]:
        wpr = k * bits // 32
        packed = torch.randint(-(2**31), 2**31, (rows, wpr), dtype=torch.int32, generator=gen)
        scales = (torch.rand(rows, k // group, generator=gen) * 0.015 + 0.005).to(torch.bfloat16)
        offsets = (-(1 << (bits - 1)) * scales.float()).to(torch.bfloat16)
        x = torch.randn(m, k, generator=gen).to(torch.bfloat16)
        mods.append((x, packed, scales, offsets, bits, k))
        total_bytes += packed.numel() * 4 + scales.numel() * 4 + m * k * 2 + m * rows * 2

    use_ref = REF_LIB.exists() and not os.environ.get("DQ_BASELINE_FORCE_PORT")
    if use_ref:
        torch.ops.load_library(str(REF_LIB))
        kind, cores = "reference", torch.get_num_threads()

        def run(x, packed, scales, offsets, bits, k):
            # reference operator: x dtype must equal the scales dtype (bf16 here)
            return torch.ops.dynquant.gemv(x, packed, scales, offsets, bits, group, k)
    else:
        sys.path.insert(0, str(HERE.parent))
        from oracle import oracle as O

        kind, cores = "port", 1

        def raw(t):
            return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()

        def run(x, packed, scales, offsets, bits, k):
            return O.c_gemv(raw(x), "bf16", packed.numpy().view(np.uint32), raw(scales), raw(offsets),
                            "bf16", O.geometry(bits, group, k))

    run(*mods[0])  # warm-up (page-in, thread pool)
    repeat = int(spec.get("repeat", 1))
    t0 = time.perf_counter()
    for _ in range(repeat):
        for mod in mods:
            run(*mod)
    seconds = time.perf_counter() - t0
    print(json.dumps({
        "kind": kind, "cores": cores, "seconds": seconds, "bytes": total_bytes * repeat,
        "gbps": total_bytes * repeat / seconds / 1e9, "modules": len(mods) * repeat,
    }))


if __name__ == "__main__":
    main()
