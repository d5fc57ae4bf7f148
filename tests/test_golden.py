"""Committed golden vectors (tests/golden/sampler_golden.json, made by tests/golden/make_golden.py):
the oracle must still reproduce them on CPU, and the CUDA library must reproduce them through the
C ABI.  Inputs are regenerated from seeds and guarded by their SHA-256."""
import importlib.util
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
G = importlib.util.module_from_spec(spec)
spec.loader.exec_module(G)

with open(os.path.join(HERE, "golden", "sampler_golden.json")) as f:
    GOLD = json.load(f)


def _probs(bits):
    return np.array(bits, np.uint32).view(np.float32)


@pytest.fixture(scope="module")
def cases():
    return G.sample_cases()


@pytest.mark.parametrize("name", sorted(GOLD["sample"]))
def test_oracle_reproduces_golden(cases, name):
    g = GOLD["sample"][name]
    now = G.golden_for(cases[name])
    assert now["inputs_sha256"] == g["inputs_sha256"], "the seeded generator no longer makes the same inputs"
    assert now["tokens"] == g["tokens"]
    assert now["paths"] == g["paths"]
    np.testing.assert_allclose(_probs(now["token_prob_f32_bits"]), _probs(g["token_prob_f32_bits"]), rtol=1e-6)


def test_oracle_reproduces_golden_spec():
    g = GOLD["spec"]["c4_spec_verify_4seq"]
    now = G.golden_spec(G.spec_case())
    assert now == g


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GOLD["sample"]))
def test_cuda_library_reproduces_golden(cases, name):
    from opentail.stingray_b200 import BatchSampler
    from tests import parity

    g = GOLD["sample"][name]
    w = cases[name]
    hist = int(np.diff(w.history_offsets).max()) if w.history_offsets is not None else 1
    bs = BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=max(hist, 1),
                      max_top_k=max(int(w.params["top_k"].max()), 1))
    out = parity.run_gpu(bs, w)
    bs.close()
    assert out["tokens"].tolist() == g["tokens"]
    assert (out["flags"].view(np.uint32) & 7).tolist() == g["paths"]
    want = _probs(g["token_prob_f32_bits"])
    sampled = np.array(g["paths"]) >= 2
    np.testing.assert_allclose(out["probs"][sampled], want[sampled], rtol=2e-5)


@pytest.mark.gpu
def test_cuda_library_reproduces_golden_spec():
    import torch
    from opentail.stingray_b200 import BatchSampler

    g = GOLD["spec"]["c4_spec_verify_4seq"]
    w = G.spec_case()
    assert w.draft_tokens.tolist() == g["draft_tokens"]
    n_seq, L, V = g["n_seq"], g["n_draft"], g["vocab"]
    bs = BatchSampler(max_rows=n_seq * (L + 1), max_vocab=V, max_history=1, max_top_k=8, max_spec_draft=L)
    out = bs.spec_verify(torch.from_numpy(w.target).cuda(), torch.from_numpy(w.draft).cuda(), w.draft_tokens,
                         w.params, w.uniforms)
    acc, corr = out["accepted"].cpu().numpy().tolist(), out["correction"].cpu().numpy().tolist()
    bs.close()
    assert acc == g["accepted"]
    assert corr == g["correction"]
