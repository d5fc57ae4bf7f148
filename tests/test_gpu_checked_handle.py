"""A handle created with STG_CHECKED=1 keeps 256 guard bytes behind each of its device buffers; after
a tour of the entry points over awkward shapes (ragged vocabularies, full capacities, bf16 with masks,
wide nuclei, speculative verification, device-resident histories, the mask cache) every guard must
still hold its pattern.  This stands in for a memory checker, which cannot be run where these tests run."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _checked(**kw):
    from opentail.stingray_b200 import BatchSampler

    os.environ["STG_CHECKED"] = "1"
    try:
        return BatchSampler(**kw)
    finally:
        del os.environ["STG_CHECKED"]


def _guards(bs):
    n, bad = C.c_int32(0), C.c_int32(0)
    rc = bs._lib.stg_debug_check_guards(bs._h, C.byref(n), C.byref(bad))
    assert rc == 0
    return n.value, bad.value


def test_guards_survive_a_tour_of_the_entry_points():
    import torch
    from opentail.stingray_b200 import workloads as W
    from tests import parity

    rows, vocab = 40, 151936
    bs = _checked(max_rows=rows, max_vocab=262144, max_history=512, max_top_k=128, max_bias=8, max_spec_draft=3,
                  max_cached_masks=3, host_logits=True)
    try:
        n0, bad0 = _guards(bs)
        assert n0 > 20 and bad0 == -1
        # mixed rows at full row capacity, histories at full length
        w = W.config2(rows=rows, seed=3)
        parity.compare(w, parity.run_gpu(bs, w, want_topk=int(w.params["top_k"].max())))
        # bf16 + masks, the widest vocabulary
        w3 = W.config3(rows=rows, seed=4)
        parity.compare(w3, parity.run_gpu(bs, w3))
        # a ragged vocabulary and host-resident inputs
        rng = np.random.default_rng(5)
        v = 151936 - 13
        x = rng.normal(0, 2.5, (rows, v)).astype(np.float32)
        p = W._params(rows, temperature=1.1, top_p=0.97)
        p["top_k"][::3] = 64
        bs.sample_rows(x, p, uniforms=rng.random(rows).astype(np.float32), want_probs=True, want_flags=True)
        bs.build_distribution(torch.from_numpy(x[:4]).cuda(), p[:4])
        # speculative verification at the draft capacity
        w4 = W.config4(n_seq=8, n_draft=3, vocab=32000, seed=6)
        bs.spec_verify(torch.from_numpy(w4.target).cuda(), torch.from_numpy(w4.draft).cuda(), torch.from_numpy(w4.draft_tokens).cuda(),
                       w4.params, torch.from_numpy(w4.uniforms).cuda())
        # device-resident histories run to their capacity and beyond
        bs.history_reset()
        pr = W._params(rows, top_k=40, repetition_penalty=1.2)
        pr["repeat_last_n"] = 64
        lg = torch.from_numpy(x).cuda()
        for r in range(rows):
            bs.history_load(r, rng.integers(0, v, 510).astype(np.int32))
        for _ in range(4):
            out = bs.sample_rows(lg, pr, uniforms=torch.from_numpy(rng.random(rows).astype(np.float32)).cuda(), history_ring=True)
            bs.history_append(out["tokens"])
        # the mask cache filled past its capacity
        words = (v + 31) // 32
        for key in (1, 2, 3, 4):
            bs.mask_cache_put(key, rng.integers(0, 1 << 32, words, dtype=np.uint64).astype(np.uint32), v)
        bs.mask_compose(np.array([[2, 3, 4]] * rows, np.uint64), v, "and")
        bs.argmax_rows(lg)
        torch.cuda.synchronize()
        n1, bad1 = _guards(bs)
        assert n1 >= n0 and bad1 == -1, f"guard of buffer {bad1} was overwritten"
    finally:
        bs.close()


def test_unchecked_handles_carry_no_guards():
    from opentail.stingray_b200 import BatchSampler

    bs = BatchSampler(max_rows=4, max_vocab=4096)
    try:
        assert _guards(bs) == (0, -1)
    finally:
        bs.close()


@pytest.mark.parametrize("drilled_pass", ["1", "2"])
def test_a_look_back_that_runs_out_costs_a_second_pass_not_the_result(drilled_pass):
    """The one wait between CTAs in the library - the look-back over the pieces of a row, in the exp
    pass (1) and in the pass over the final probabilities (2) - is bounded.  The drill makes it run out
    without any fault: piece 0 of every row withholds its flag in the drilled pass and the wait gives
    up after 64 polls, so every later piece times out, flags its row, and the row kernel redoes the row.  Tokens and probabilities must still be the oracle's, every
    full-vocabulary row must report the second pass, and the handle must keep working."""
    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import workloads as W
    from tests import parity

    w = W.config2(rows=24, seed=11)
    os.environ["STG_LOOKBACK_DRILL"] = drilled_pass
    try:
        bs = BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=512, max_top_k=128)
    finally:
        del os.environ["STG_LOOKBACK_DRILL"]
    try:
        for _ in range(2):
            gpu = parity.run_gpu(bs, w, want_topk=int(w.params["top_k"].max()))
            parity.compare(w, gpu)
            flags = gpu["flags"].view(np.uint32)
            full = (flags & 7) == 3
            assert full.any() and ((flags[full] >> 8) & 1).all(), "every full-vocabulary row should have been redone"
        assert bs.stats()["reread_rows"] >= int(full.sum())
    finally:
        bs.close()
