"""Hardware-limit probes for the GEMM pipelines (csrc/rd_probe.cu).

    python -m gpu_ragged_dot_b200.probe [mma|tma|sync|pair|all]

Builds ``rd_probe`` next to this file with nvcc for sm_100a (no GPU needed to build) and runs it on
GPU 0.  The probes time the instructions the kernels are made of -- tcgen05.mma by operand layout
and CTA group, tiled TMA loads by box shape, the synchronisation instructions of the MMA loop, the
signalling between the two CTAs of a pair -- so a kernel's figures can be read against what one
SM can do at best.  Nothing in the library uses the probe.
"""

from __future__ import annotations

import os
import subprocess
import sys

from . import build as rd_build

PROBE_PATH = os.path.join(rd_build.PKG_DIR, "rd_probe")
SOURCE = os.path.join(rd_build.CSRC_DIR, "rd_probe.cu")


def build_probe(force: bool = False) -> str:
    deps = [SOURCE, os.path.join(rd_build.CSRC_DIR, "rd_ptx.cuh")]
    if (not force and os.path.exists(PROBE_PATH)
            and all(os.path.getmtime(d) <= os.path.getmtime(PROBE_PATH) for d in deps)):
        return PROBE_PATH
    cmd = [rd_build._nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-o", PROBE_PATH, SOURCE, "-lcuda"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    return PROBE_PATH


def main(argv) -> int:
    path = build_probe(force="--force" in argv)
    which = [a for a in argv if not a.startswith("-")] or ["all"]
    return subprocess.call([path, which[0]])


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
