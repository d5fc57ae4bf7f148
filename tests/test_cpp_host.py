"""The C++ wrapper header compiles, links against the C-ABI library and behaves: without a GPU it must
refuse to create a sampler (no CPU fallback); with one it runs a small batch (gpu-marked test)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build_host_check():
    from opentail.stingray_b200 import build as B

    lib = B.build()
    libdir = os.path.dirname(lib)
    out = os.path.join(ROOT, "tests", "cpp", "_build", "host_check")
    src = os.path.join(ROOT, "tests", "cpp", "host_check.cpp")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    newest = max(os.path.getmtime(p) for p in (src, lib, os.path.join(ROOT, "include", "stingray_sampler.hpp"),
                                               os.path.join(ROOT, "include", "stingray_sampler.h")))
    if not os.path.exists(out) or os.path.getmtime(out) < newest:
        subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), src, "-o", out,
                        "-L", libdir, "-lstingray_sampler", f"-Wl,-rpath,{libdir}"], check=True)
    return out


def _run(exe):
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    return r.returncode, r.stdout


def test_cpp_wrapper_refuses_without_a_device():
    import torch

    exe = _build_host_check()
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    code, out = _run(exe)
    assert code == 0, out
    assert "creation refused" in out


@pytest.mark.gpu
def test_cpp_wrapper_samples_a_small_batch():
    code, out = _run(_build_host_check())
    assert code == 0, out
    assert "host_check: ok" in out
