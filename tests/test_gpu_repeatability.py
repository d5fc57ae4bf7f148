"""Repeatability: the same batch on the same handle must give the same tokens, flags and probabilities
every time, whatever the handle ran before.  The sweep's batches are repeated in random order on one
handle, on the legacy default stream (direct launches) and on a stream of the test's own (where the
library replays repeated steps as CUDA graphs); the first run of each batch is checked against the
oracle, every later run against the first.  Results that depend on what a CTA processed before, or
on how three streams happened to interleave, show up here and nowhere else."""
import numpy as np
import pytest

from tests import parity
from tests.test_gpu_random_sweep import _workload

pytestmark = pytest.mark.gpu

CASES = [0, 1, 2, 3, 4, 9, 11, 69, 78, 141, 149, 171, 195]


@pytest.mark.parametrize("own_stream", [False, True])
def test_repeated_batches_in_random_order(own_stream):
    import torch
    from opentail.stingray_b200 import BatchSampler

    bs = BatchSampler(max_rows=64, max_vocab=262144, max_history=1024, max_top_k=512)
    st = torch.cuda.Stream() if own_stream else torch.cuda.current_stream()
    try:
        with torch.cuda.stream(st):
            ws = {it: _workload(it) for it in CASES}
            devs = {it: parity.to_device(ws[it]) for it in CASES}
            first = {}
            rng = np.random.default_rng(7)
            for rep in range(25):
                for it in (rng.permutation(CASES) if rep else CASES):
                    it = int(it)
                    gpu = parity.run_gpu(bs, ws[it], devs[it], want_topk=512)
                    if it not in first:
                        parity.compare(ws[it], gpu)
                        first[it] = gpu
                        continue
                    for key in ("tokens", "flags", "probs"):
                        np.testing.assert_array_equal(gpu[key].view(np.uint32), first[it][key].view(np.uint32),
                                                      err_msg=f"case {it}, repeat {rep}: {key} differ from the first run")
    finally:
        bs.close()
