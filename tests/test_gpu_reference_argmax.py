"""stg_argmax_rows against the reference's own device kernel, llm_argmax_rows
(src/OpenTail.Stingray.Cuda/CudaTextKernels.cs:388-445), compiled from the reference's source text into
oracle/_ref/ at build time: the (index, value) pairs must be identical, ties and fully masked rows
included (CudaGpuArgmaxParityTests.cs:31-38).  Skipped where that library was not built."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref_argmax.so")


@pytest.mark.skipif(not os.path.exists(SO), reason="oracle/_ref/libref_argmax.so was not built (no reference tree at build time)")
@pytest.mark.parametrize("rows,vocab", [(1, 151936), (7, 32000), (64, 262144), (256, 151936), (3, 1000)])
def test_pairs_identical_to_the_reference_kernel(rows, vocab):
    import torch
    from opentail.stingray_b200 import BatchSampler

    lib = ctypes.CDLL(SO)
    lib.ref_argmax_rows.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    rng = np.random.default_rng(rows * 31 + vocab)
    x = rng.normal(0, 3, (rows, vocab)).astype(np.float32)
    x[0, vocab // 3] = x[0].max()          # a tie: the lower index wins
    x[0, vocab // 3 + 17] = x[0].max()
    if rows > 2:
        x[2, :] = -np.inf                  # nothing finite: token 0
        x[1, 5:] = x[1, 5]                 # a long plateau
    xd = torch.from_numpy(x).cuda()
    bs = BatchSampler(max_rows=rows, max_vocab=vocab, max_history=1, max_top_k=1)
    try:
        idx, val = bs.argmax_rows(xd)
        pairs = torch.empty((rows, 2), dtype=torch.int32, device="cuda")
        rc = lib.ref_argmax_rows(xd.data_ptr(), rows, vocab, vocab, pairs.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(pairs[:, 0], idx)
        finite = torch.isfinite(val)
        assert torch.equal(pairs[:, 1][finite], val.view(torch.int32)[finite])
    finally:
        bs.close()
