"""Builds the CUDA library in-tree with nvcc for sm_100a.

    python -m opentail.stingray_b200.build [--force] [-v]

produces ``opentail/stingray_b200/libstingray_sampler.so`` next to this file (the shared
library a host binds through the C ABI declared in ``include/stingray_sampler.h``).  Every
translation unit is compiled to an object file of its own (in parallel, only when it or a header
changed) and the objects are linked into the shared library.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_build")
OUT = os.path.join(HERE, "libstingray_sampler.so")
INCLUDE = os.path.join(HERE, "..", "..", "include", "stingray_sampler.h")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = [*ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden"]
LFLAGS = [*ARCH, "-shared", "-cudart", "shared", "-Xcompiler", "-fPIC"]


def sources():
    return sorted(n for n in os.listdir(CSRC) if n.endswith(".cu"))


def _headers_mtime() -> float:
    t = os.path.getmtime(INCLUDE)
    for name in os.listdir(CSRC):
        if name.endswith((".h", ".cuh", ".inc")):
            t = max(t, os.path.getmtime(os.path.join(CSRC, name)))
    return t


def _compile(nvcc: str, name: str, verbose: bool):
    src = os.path.join(CSRC, name)
    obj = os.path.join(OBJ, name[:-3] + ".o")
    cmd = [nvcc, *CFLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    return name, res.returncode, res.stdout + res.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ, exist_ok=True)
    hdr = _headers_mtime()
    todo = []
    for name in sources():
        obj = os.path.join(OBJ, name[:-3] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(hdr, os.path.getmtime(os.path.join(CSRC, name))):
            todo.append(name)
    objs = [os.path.join(OBJ, n[:-3] + ".o") for n in sources()]
    if not todo and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(o) for o in objs):
        return OUT
    with ThreadPoolExecutor(max(1, min(len(todo), os.cpu_count() or 1))) as ex:
        for name, rc, log in ex.map(lambda n: _compile(nvcc, n, verbose), todo):
            if verbose or rc != 0:
                sys.stderr.write(f"---- {name}\n{log}")
            if rc != 0:
                raise RuntimeError(f"nvcc failed compiling {name}")
    res = subprocess.run([nvcc, *LFLAGS, "-o", OUT, *objs, "-ldl"], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed linking libstingray_sampler.so")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
