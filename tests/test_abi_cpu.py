"""CPU-side checks of the boundary: the C-ABI library loads and exports every symbol declared in
include/stingray_sampler.h, struct sizes agree, and argument errors are reported as status codes
without touching a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from opentail.stingray_b200 import build as B
    from opentail.stingray_b200 import _native as N

    B.build()
    return N.load(), N


def test_header_symbols_are_exported():
    lib, N = _lib()
    header = open(os.path.join(ROOT, "include", "stingray_sampler.h")).read()
    declared = set(re.findall(r"STG_API\s+\w+\s+\**\s*(stg_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(N.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert lib.stg_abi_version() == 2


def test_struct_layouts_match_the_header():
    _, N = _lib()
    assert C.sizeof(N.StgRowParams) == 32
    assert C.sizeof(N.StgConfig) == 40
    assert C.sizeof(N.StgSampleBatch) == 176
    assert C.sizeof(N.StgStats) == 128
    from opentail.stingray_b200.sampler import PARAMS_DTYPE

    assert PARAMS_DTYPE.itemsize == C.sizeof(N.StgRowParams)


def test_create_rejects_bad_config_without_a_device():
    lib, N = _lib()
    h = C.c_void_p()
    assert lib.stg_create(None, C.byref(h)) == 1
    cfg = N.StgConfig(C.sizeof(N.StgConfig), 0, 0, 1000, 0, 0, 0, 0, 0, 0)
    assert lib.stg_create(C.byref(cfg), C.byref(h)) == 1  # max_rows must be positive
    cfg = N.StgConfig(C.sizeof(N.StgConfig), 0, 4, 1000, 8000, 4000, 0, 0, 0, 0)
    assert lib.stg_create(C.byref(cfg), C.byref(h)) == 3  # top_k + history beyond 8192
    buf = C.create_string_buffer(256)
    lib.stg_last_error(None, buf, 256)
    assert b"8192" in buf.value


def test_no_cpu_fallback_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    lib, N = _lib()
    h = C.c_void_p()
    cfg = N.StgConfig(C.sizeof(N.StgConfig), 0, 4, 1000, 16, 16, 0, 0, 0, 0)
    assert lib.stg_create(C.byref(cfg), C.byref(h)) == 7  # STG_ERR_NO_DEVICE
    from opentail.stingray_b200 import BatchSampler, StingrayError

    with pytest.raises(StingrayError):
        BatchSampler(4, 1000)
