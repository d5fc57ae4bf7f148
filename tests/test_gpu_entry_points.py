"""GPU parity tests of the managed entry points beside Sample / Greedy / BuildFilteredDistribution:
SampleWithDistribution, SampleFromProbs and ResampleResidual (Sampler.cs:172-199, :587-618), through
the C ABI and through the host mirror, against the reference's literals (SamplerTests.cs:403-442)
and the CPU oracle on full-vocabulary rows."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import parity

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bs():
    from opentail.stingray_b200 import BatchSampler

    s = BatchSampler(max_rows=256, max_vocab=151936, max_history=512, max_top_k=512)
    yield s
    s.close()


def test_sample_with_distribution_reference_literal():
    from opentail.stingray_b200 import Random, Sampler, SamplingParams

    logits = np.array([0.0, 12.0, 0.0, 0.0], np.float32)
    probs = np.zeros(4, np.float32)
    rng = Random(7)
    tok = Sampler.SampleWithDistribution(logits, SamplingParams(Temperature=0.1), probs, rng)
    assert tok == 1 and probs[1] > 0.99 and abs(float(probs.sum()) - 1.0) < 1e-5
    assert rng.draws == 1
    # temperature 0: one-hot at the (penalised) arg-max, no draw
    rng = Random(1)
    tok = Sampler.SampleWithDistribution(np.array([5.0, 4.9, 1.0], np.float32),
                                         SamplingParams(Temperature=0.0, PresencePenalty=1.0, PreviousTokens=[0]), probs[:3], rng)
    assert tok == 1 and list(probs[:3]) == [0.0, 1.0, 0.0] and rng.draws == 0


def test_sample_with_distribution_forces_the_full_pipeline(bs):
    import torch
    from opentail.stingray_b200 import workloads as W

    rng = np.random.default_rng(77)
    rows, vocab = 12, 151936
    logits = rng.normal(0, 2.5, (rows, vocab)).astype(np.float32)
    p = W._params(rows)
    p["temperature"] = rng.uniform(0.5, 1.2, rows).astype(np.float32)
    p["top_k"] = [50, 0, 200, 50, 0, 20, 50, 0, 100, 3, 50, 0]      # 0 < top_k < V would take the fast path in Sample
    p["top_p"] = [0.9, 0.95, 1.0, 0.8, 1.0, 0.9, 0.99, 0.9, 0.9, 1.0, 0.5, 0.9]
    p["min_p"] = [0.0, 0.0, 0.02, 0.0, 0.0, 0.0, 0.0, 0.05, 0.0, 0.0, 0.0, 0.0]
    p["frequency_penalty"] = 0.5
    hist = rng.integers(0, vocab, (rows, 64)).astype(np.int32)
    u = W.uniforms24(rng, rows)
    tok, probs = bs.sample_with_distribution(torch.from_numpy(logits).cuda(), p, history_ids=torch.from_numpy(hist.reshape(-1)).cuda(),
                                             history_offsets=(np.arange(rows + 1) * 64).astype(np.int32),
                                             uniforms=torch.from_numpy(u).cuda())
    tok, probs = tok.cpu().numpy(), probs.cpu().numpy()
    boundary = 0
    for r in range(rows):
        op = orc.OrcParams(*[p[r][n].item() for n in p.dtype.names])
        want_tok, want, tr = orc.sample_with_distribution(logits[r], op, float(u[r]), history=hist[r])
        assert np.array_equal(probs[r] > 0, want > 0), f"row {r}: support differs"
        np.testing.assert_allclose(probs[r], want, rtol=1e-5, atol=1e-30, err_msg=f"row {r}")
        if tok[r] != want_tok:
            assert tr.margin <= parity.BOUNDARY, f"row {r}: token {tok[r]} != {want_tok}"
            boundary += 1
    assert boundary <= 1


def test_sample_from_probs_matches_oracle(bs):
    import torch

    rng = np.random.default_rng(5)
    rows, vocab = 16, 151936
    x = rng.normal(0, 3, (rows, vocab)).astype(np.float32)
    probs = np.stack([orc.build_filtered_distribution(x[r], orc.make_params(temperature=0.9, top_p=0.95 if r % 2 else 1.0))[0] for r in range(rows)])
    u = rng.random(rows).astype(np.float32)
    u[0] = 0.0          # r == 0: token 0 whatever its probability (Sampler.cs:566-571)
    u[1] = 0.99999994   # just below 1: may run off the end of a rounded CDF
    tok, fl = bs.sample_from_probs(torch.from_numpy(probs).cuda(), u)
    tok, fl = tok.cpu().numpy(), fl.cpu().numpy().view(np.uint32)
    for r in range(rows):
        want, tr = orc.sample_from_probs(probs[r], float(u[r]))
        assert tok[r] == want, f"row {r}"
        assert bool(fl[r] & (1 << 5)) == bool(tr.fallback), f"row {r}: fallback flag"
    from opentail.stingray_b200 import Random, Sampler

    assert Sampler.SampleFromProbs(np.array([0.0, 0.0, 1.0, 0.0], np.float32), Random(3)) == 2


def test_resample_residual_reference_literals_and_oracle(bs):
    import torch
    from opentail.stingray_b200 import Random, Sampler

    # concentrated residual: p on {1, 2}, q takes all of token 1 -> always token 2 (SamplerTests.cs:416-424)
    p = np.tile(np.array([0.0, 0.5, 0.5, 0.0], np.float32), (200, 1))
    q = np.tile(np.array([0.0, 1.0, 0.0, 0.0], np.float32), (200, 1))
    u = np.random.default_rng(3).random((200, 2)).astype(np.float32)
    tok, fl = bs.resample_residual(torch.from_numpy(p).cuda(), torch.from_numpy(q).cuda(), u)
    assert (tok.cpu().numpy() == 2).all() and (fl.cpu().numpy() == 0).all()
    # empty residual: falls back to a draw from p (SamplerTests.cs:426-435)
    e = np.full((8, 4), 0.25, np.float32)
    ue = np.random.default_rng(5).random((8, 2)).astype(np.float32)
    tok, fl = bs.resample_residual(torch.from_numpy(e).cuda(), torch.from_numpy(e).cuda(), ue)
    tok, fl = tok.cpu().numpy(), fl.cpu().numpy().view(np.uint32)
    for r in range(8):
        want, used, _ = orc.resample_residual(e[r], e[r], float(ue[r, 0]), float(ue[r, 1]))
        assert tok[r] == want and (fl[r] & (1 << 8))
    with pytest.raises(ValueError):   # SamplerTests.cs:437-442
        Sampler.ResampleResidual(np.zeros(4, np.float32), np.zeros(3, np.float32), Random(1))
    assert Sampler.ResampleResidual(p[0], q[0], Random(9)) == 2
    # full-vocabulary distributions built by the oracle
    rng = np.random.default_rng(11)
    rows, vocab = 12, 151936
    d = rng.normal(0, 3, (rows, vocab)).astype(np.float32)
    t = d + rng.normal(0, 0.5, (rows, vocab)).astype(np.float32)
    par = orc.make_params(temperature=1.0)
    P = np.stack([orc.build_filtered_distribution(t[r], par)[0] for r in range(rows)])
    Q = np.stack([orc.build_filtered_distribution(d[r], par)[0] for r in range(rows)])
    u = rng.random((rows, 2)).astype(np.float32)
    tok, _ = bs.resample_residual(torch.from_numpy(P).cuda(), torch.from_numpy(Q).cuda(), u)
    tok = tok.cpu().numpy()
    for r in range(rows):
        want, used, tr = orc.resample_residual(P[r], Q[r], float(u[r, 0]), float(u[r, 1]))
        assert tok[r] == want or tr.margin <= parity.BOUNDARY, f"row {r}: {tok[r]} != {want}"


def test_calls_alternating_between_streams_are_ordered(bs):
    """Two streams driving one handle in turn: every call must see the workspace as the previous call
    left it, so the results equal those of the same calls on a single stream."""
    import torch
    from opentail.stingray_b200 import workloads as W

    ws = [W.config2(rows=48, seed=40 + i) for i in range(4)]
    devs = [parity.to_device(w) for w in ws]
    torch.cuda.synchronize()

    def run(streams):
        outs = []
        for i in range(8):
            w, d = ws[i % 4], devs[i % 4]
            st = streams[i % len(streams)]
            outs.append(bs.sample_rows(d["logits"], w.params, uniforms=d["uniforms"], history_ids=d["history_ids"],
                                       history_offsets=w.history_offsets, want_probs=True, stream=st))
        torch.cuda.synchronize()
        return [(o["tokens"].cpu().numpy(), o["probs"].cpu().numpy()) for o in outs]

    one = run([torch.cuda.Stream()])
    two = run([torch.cuda.Stream(), torch.cuda.Stream()])
    for (t1, p1), (t2, p2) in zip(one, two):
        assert np.array_equal(t1, t2) and np.array_equal(p1, p2)
