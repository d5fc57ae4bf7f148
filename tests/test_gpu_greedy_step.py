"""A step of plain arg-max rows only runs as one launch (stg_flat_greedy.cu).  Its results must be the
oracle's Greedy (Sampler.cs:83-99: highest logit, lowest index on ties, token 0 for a row without a
finite value), and it must leave the per-row state as the other forms of the step expect it and find
it as they leave it."""
import numpy as np
import pytest

from tests import parity

pytestmark = pytest.mark.gpu


def _greedy_workload(seed, rows, vocab, bf16=False, ties=False, mask_density=None):
    from opentail.stingray_b200 import workloads as W

    rng = np.random.default_rng(seed)
    logits = rng.normal(0, 3.0, (rows, vocab)).astype(np.float32)
    if ties:
        logits = np.round(logits)  # many equal maxima: the lowest index must win
    mask = None
    if mask_density is not None:
        words = (vocab + 31) // 32
        bits = rng.random((rows, words * 32)) < mask_density
        bits[0, :] = False  # row 0 fully masked: token 0, STG_ROW_FULLY_MASKED
        mask = np.packbits(bits, axis=1, bitorder="little").view(np.uint32)
    lg = W.to_bf16_bits(logits) if bf16 else logits
    return W.SampleWorkload("greedy", np.ascontiguousarray(lg), W._params(rows, temperature=0.0),
                            W.uniforms24(rng, rows), None, None, mask)


@pytest.mark.parametrize("vocab,bf16,ties,dens", [(151936, False, False, None), (32000, True, True, None),
                                                 (50264, False, True, 0.3), (262144, True, False, 0.01),
                                                 (16384, False, False, None), (4104, False, True, 0.9)])
def test_all_greedy_step_is_one_launch_and_matches_oracle(vocab, bf16, ties, dens):
    from opentail.stingray_b200 import BatchSampler

    w = _greedy_workload(vocab, 40, vocab, bf16, ties, dens)
    bs = BatchSampler(max_rows=64, max_vocab=vocab, max_history=8, max_top_k=8)
    try:
        dev = parity.to_device(w)
        for _ in range(3):  # the kernel must leave the state it starts from
            before = bs.stats()["kernel_launches"]
            gpu = parity.run_gpu(bs, w, dev)
            assert bs.stats()["kernel_launches"] - before == 1
            parity.compare(w, gpu)
            if dens is not None:
                assert gpu["tokens"][0] == 0 and (gpu["flags"].view(np.uint32)[0] >> 6) & 1
    finally:
        bs.close()


def test_greedy_step_between_other_forms_of_the_step():
    """all-greedy, mixed (greedy + top-k + full-vocabulary rows), all-greedy again, on one handle."""
    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import workloads as W

    vocab = 50264
    g = _greedy_workload(5, 32, vocab, ties=True)
    mixed = W.SampleWorkload("mixed", g.logits, W._params(32), g.uniforms, None, None, None)
    rng = np.random.default_rng(9)
    mixed.params["temperature"] = rng.choice([0.0, 0.8], 32).astype(np.float32)
    mixed.params["top_k"] = rng.choice([0, 40], 32)
    mixed.params["top_p"] = rng.choice([1.0, 0.9], 32).astype(np.float32)
    bs = BatchSampler(max_rows=32, max_vocab=vocab, max_history=8, max_top_k=64)
    try:
        dev = parity.to_device(g)
        for w in (g, mixed, g, mixed, mixed, g, g):
            gpu = parity.run_gpu(bs, w, dev)
            stats = parity.compare(w, gpu, check_topk=False)
            assert stats["mismatch"] == stats["boundary_draws"] <= 1
        idx, val = bs.argmax_rows(dev["logits"])
        want = g.logits.argmax(axis=1)
        np.testing.assert_array_equal(idx.cpu().numpy(), want)
        np.testing.assert_array_equal(val.cpu().numpy(), g.logits[np.arange(32), want])
        gpu = parity.run_gpu(bs, g, dev)
        parity.compare(g, gpu)
    finally:
        bs.close()
