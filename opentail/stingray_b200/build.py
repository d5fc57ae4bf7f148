"""Builds the CUDA library in-tree with nvcc for sm_100a.

    python -m opentail.stingray_b200.build

produces ``opentail/stingray_b200/libstingray_sampler.so`` next to this file (the shared
library a host binds through the C ABI declared in ``include/stingray_sampler.h``).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libstingray_sampler.so")
SOURCES = ["stg_kernels.cu", "stg_api.cu", "stg_spec.cu", "stg_spec_kernels.cu", "stg_static.cu", "stg_mask.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared", "-cudart", "shared",
]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    for name in os.listdir(CSRC):
        if os.path.getmtime(os.path.join(CSRC, name)) > t:
            return True
    inc = os.path.join(HERE, "..", "..", "include", "stingray_sampler.h")
    return os.path.getmtime(inc) > t


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-o", OUT, *[os.path.join(CSRC, s) for s in SOURCES], "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libstingray_sampler.so")
    if verbose:
        print(res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
