"""TEST INFRASTRUCTURE ONLY.  Builds ``oracle/_ref/libref_argmax.so``: the reference's own CUDA
arg-max kernel (``llm_argmax_rows``, held as CUDA C text inside
``src/OpenTail.Stingray.Cuda/CudaTextKernels.cs`` and compiled there by NVRTC at run time), compiled
here with nvcc so that the benchmark can time it beside ``stg_argmax_rows`` and the tests can compare
both.  The kernel text is extracted from the reference tree where it lies; nothing of it is kept in
this repository (``oracle/_ref/`` is build output).

    python oracle/build_ref_argmax.py [/path/to/reference]

Without a reference tree the script leaves a previously built library alone and reports that it
could not build; callers treat the library as optional.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
SO = os.path.join(OUT_DIR, "libref_argmax.so")
REL = os.path.join("src", "OpenTail.Stingray.Cuda", "CudaTextKernels.cs")
# the reference checkout: STG_REFERENCE_ROOT, else a directory `reference` beside this repository
DEFAULT_REFERENCE = os.environ.get("STG_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def extract(cs_text: str) -> str:
    """The sentinel #define and the llm_argmax_rows kernel, un-escaped from the C# raw string
    (inside it a double quote is written twice)."""
    m = re.search(r"^#define STINGRAY_ARGMAX_NEG_INF[^\n]*\n", cs_text, re.M)
    k = re.search(r'^extern ""C"" __global__ void llm_argmax_rows\(.*?^\}\n', cs_text, re.M | re.S)
    if not m or not k:
        raise RuntimeError("llm_argmax_rows not found in the reference source")
    return (m.group(0) + "\n" + k.group(0)).replace('""', '"')


def build(reference_root: str | None = None) -> str | None:
    reference_root = reference_root or DEFAULT_REFERENCE
    src = os.path.join(reference_root, REL)
    if not os.path.exists(src):
        return SO if os.path.exists(SO) else None
    os.makedirs(OUT_DIR, exist_ok=True)
    inc = os.path.join(OUT_DIR, "llm_argmax_rows.inc")
    with open(src, encoding="utf-8") as f:
        text = extract(f.read())
    with open(inc, "w", encoding="utf-8") as f:
        f.write(text)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    # the reference compiles for the detected device's plain architecture (CudaBackend.cs:7195)
    cmd = [nvcc, "-arch=sm_100", "-O3", "-shared", "-Xcompiler", "-fPIC", "-cudart", "shared",
           "-o", SO, os.path.join(HERE, "ref_argmax_wrapper.cu")]
    subprocess.run(cmd, check=True, capture_output=True)
    return SO


if __name__ == "__main__":
    out = build(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out or "reference tree not present and no earlier build: nothing built")
