"""The allocation-free arg-max entry point (for hosts that may not call cudaMalloc where they need
the result) must give exactly what the regular entry point gives.  Runs last so that a run that
stops at the first failure has already exercised everything else."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _static_argmax(x):
    """Calls stg_argmax_rows_static through the C ABI on a CUDA tensor; returns (index, value)."""
    import torch
    from opentail.stingray_b200 import _native as N

    lib = N.load()
    rows, width = x.shape
    out = torch.empty((rows, 2), dtype=torch.int32, device=x.device)
    dtype = N.DTYPE_BF16 if x.dtype == torch.bfloat16 else N.DTYPE_F32
    rc = lib.stg_argmax_rows_static(x.data_ptr(), dtype, rows, width, x.stride(0) if rows > 1 else width,
                                    out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, f"stg_argmax_rows_static returned {rc}"
    torch.cuda.synchronize()
    return out[:, 0].cpu().numpy(), out[:, 1].view(torch.float32).cpu().numpy()


def test_static_argmax_matches_regular_entry_point_twice_in_a_row():
    import torch
    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import _native as N
    from oracle import oracle as orc

    rng = np.random.default_rng(2024)
    bs = BatchSampler(max_rows=64, max_vocab=152064, max_history=1, max_top_k=1)
    try:
        for call, (rows, vocab) in enumerate([(5, 152064), (64, 40000)]):
            a = rng.normal(0, 3, (rows, vocab)).astype(np.float32)
            a[0, 17] = a[0, 9000] = 99.0          # a tie: the lower index must win in both
            x = torch.from_numpy(a).cuda()
            ref_i, ref_v = bs.argmax_rows(x)
            got_i, got_v = _static_argmax(x)
            assert np.array_equal(got_i, ref_i.cpu().numpy()), f"call {call}: indices differ"
            assert np.array_equal(got_v.view(np.uint32), ref_v.cpu().numpy().view(np.uint32)), f"call {call}: values differ"
            assert got_i[0] == 17
            # and against the CPU restatement of Sampler.Greedy, row by row
            want = np.array([orc.greedy(a[r]) for r in range(rows)])
            assert np.array_equal(got_i, want), f"call {call}: indices differ from the oracle's"
        xb = torch.from_numpy(rng.normal(0, 3, (3, 70001)).astype(np.float32)).cuda().to(torch.bfloat16)
        ref_i, _ = bs.argmax_rows(xb)
        got_i, _ = _static_argmax(xb)           # odd width: unaligned rows take the scalar-load path
        assert np.array_equal(got_i, ref_i.cpu().numpy())
        # beyond the fixed scratch the call is refused, not truncated
        lib = N.load()
        big = torch.zeros((1, 8), device="cuda")
        assert lib.stg_argmax_rows_static(big.data_ptr(), 0, 5000, 8, 8, big.data_ptr(), None) == 3
    finally:
        bs.close()
