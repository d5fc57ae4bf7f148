"""Randomised parity sweep: every sampling knob, mask densities, histories, tie-heavy and bf16 logits,
vocabulary sizes that are and are not multiples of the tile sizes - the CUDA library against the
oracle, row by row.  Seeds are fixed; the cases were chosen because earlier builds failed on them."""
import numpy as np
import pytest

from tests import parity

pytestmark = pytest.mark.gpu


def _workload(it):
    from opentail.stingray_b200 import workloads as W

    rng = np.random.default_rng(1000 + it)
    rows = 48
    vocab = int(rng.choice([4097, 32000, 50257, 151936, 200003, 262144]))
    sigma = float(rng.choice([0.5, 2.0, 3.5, 6.0]))
    logits = rng.normal(0, sigma, (rows, vocab)).astype(np.float32)
    if it % 3 == 0:
        logits = np.round(logits * 4) / 4  # ties
    bf16 = it % 4 == 1
    p = W._params(rows)
    p["temperature"] = rng.choice([0.0, 0.3, 0.7, 1.0, 1.5], rows).astype(np.float32)
    p["top_k"] = rng.choice([0, 0, 1, 5, 40, 300], rows)
    p["top_p"] = rng.choice([1.0, 0.5, 0.9, 0.99, 0.9999], rows).astype(np.float32)
    p["min_p"] = rng.choice([0.0, 0.0, 0.01, 0.2], rows).astype(np.float32)
    p["repetition_penalty"] = rng.choice([1.0, 1.1, 0.8], rows).astype(np.float32)
    p["presence_penalty"] = rng.choice([0.0, 0.5, -0.5], rows).astype(np.float32)
    p["frequency_penalty"] = rng.choice([0.0, 0.3], rows).astype(np.float32)
    p["repeat_last_n"] = rng.choice([0, 16, 64], rows)
    H = int(rng.choice([0, 7, 300, 700]))
    hist = [rng.integers(0, vocab, H) for _ in range(rows)] if H else None
    mask = None
    if it % 2 == 0:
        words = (vocab + 31) // 32
        dens = float(rng.choice([0.01, 0.3, 0.9]))
        bits = rng.random((rows, words * 32)) < dens
        bits[:, :3] = True
        mask = np.packbits(bits, axis=1, bitorder="little").view(np.uint32)
    lg = W.to_bf16_bits(logits) if bf16 else logits
    ids = off = None
    if hist is not None:
        ids = np.concatenate(hist).astype(np.int32); off = np.arange(rows + 1, dtype=np.int32) * H
    w = W.SampleWorkload("s", np.ascontiguousarray(lg), p, W.uniforms24(rng, rows), ids, off, mask)
    return w
    return w


@pytest.fixture(scope="module")
def bs():
    from opentail.stingray_b200 import BatchSampler

    s = BatchSampler(max_rows=64, max_vocab=262144, max_history=1024, max_top_k=512)
    yield s
    s.close()


@pytest.mark.parametrize("it", [0, 1, 2, 3, 4, 9, 11, 69, 78, 141, 149, 171, 195])
def test_random_batch_matches_oracle(bs, it):
    w = _workload(it)
    gpu = parity.run_gpu(bs, w, want_topk=512)
    stats = parity.compare(w, gpu)
    assert stats["mismatch"] == stats["boundary_draws"] <= 1
