"""GPU parity tests: the CUDA library, called through its C ABI, against the CPU oracle."""
import math

import numpy as np
import pytest

from oracle import oracle as orc
from tests import parity

pytestmark = pytest.mark.gpu
NEG = -math.inf


@pytest.fixture(scope="module")
def bs():
    from opentail.stingray_b200 import BatchSampler

    s = BatchSampler(max_rows=256, max_vocab=262144, max_history=1024, max_top_k=1024, max_bias=64)
    yield s
    s.close()


def _params(rows, **kw):
    from opentail.stingray_b200 import workloads as W

    return W._params(rows, **kw)


def _wl(logits, params, uniforms, hist=None, mask=None):
    from opentail.stingray_b200 import workloads as W

    ids = off = None
    if hist is not None:
        ids = np.concatenate([np.asarray(h, np.int32) for h in hist]) if len(hist) else np.zeros(0, np.int32)
        off = np.concatenate([[0], np.cumsum([len(h) for h in hist])]).astype(np.int32)
    return W.SampleWorkload("t", np.ascontiguousarray(logits), params, np.asarray(uniforms, np.float32), ids, off, mask)


# ---- CudaGpuArgmaxParityTests.cs:57-176 through stg_argmax_rows --------------------------------
@pytest.mark.parametrize("n", [1, 2, 3, 255, 256, 257, 1000, 65536, 152064, 262144])
def test_argmax_sizes_positions(bs, n):
    import torch

    rng = np.random.default_rng(1234 + n)
    a = (rng.random(n) * 20 - 10).astype(np.float32)
    cases = [a]
    for pos in (0, n // 2, n - 1):
        b = a.copy()
        b[pos] = 1000.0 + pos
        cases.append(b)
    x = torch.from_numpy(np.stack(cases)).cuda()
    idx, val = bs.argmax_rows(x)
    idx, val = idx.cpu().numpy(), val.cpu().numpy()
    for r, c in enumerate(cases):
        assert idx[r] == orc.greedy(c)
        assert val[r].view(np.uint32) == c[idx[r]].view(np.uint32)


def test_argmax_ties_constant_negative_rows(bs):
    import torch

    a = np.full(5000, -1.0, np.float32)
    a[700] = 5.0
    a[300] = 5.0
    idx, _ = bs.argmax_rows(torch.from_numpy(a[None]).cuda())
    assert int(idx[0]) == 300
    idx, _ = bs.argmax_rows(torch.full((1, 8192), 3.5, device="cuda"))
    assert int(idx[0]) == 0
    rng = np.random.default_rng(99)
    neg = (-rng.random(4096) * 50 - 1).astype(np.float32)
    idx, val = bs.argmax_rows(torch.from_numpy(neg[None]).cuda())
    assert int(idx[0]) == orc.greedy(neg) and float(val[0]) == neg.max()


@pytest.mark.parametrize("vocab", [1024, 152064])
@pytest.mark.parametrize("rows", [1, 2, 4, 8])
def test_argmax_rows_batched(bs, rows, vocab):
    import torch

    rng = np.random.default_rng(555 + rows * 31 + vocab)
    flat = (rng.random((rows, vocab)) * 10 - 5).astype(np.float32)
    for r in range(rows):
        pos = (r * 37) % vocab
        flat[r, pos] = 50.0 + r
        if vocab > 100:
            flat[r, (pos + 50) % vocab] = 50.0 + r
    idx, val = bs.argmax_rows(torch.from_numpy(flat).cuda())
    for r in range(rows):
        assert int(idx[r]) == orc.greedy(flat[r])
        assert float(val[r]) == flat[r].max()


def test_argmax_strided_and_bf16_rows(bs):
    import torch

    rng = np.random.default_rng(5)
    wide = torch.from_numpy(rng.normal(0, 3, (6, 3001)).astype(np.float32)).cuda()
    idx, _ = bs.argmax_rows(wide, valid_len=2999)  # unaligned stride: scalar-load path
    ref = wide[:, :2999].cpu().numpy()
    for r in range(6):
        assert int(idx[r]) == orc.greedy(ref[r])
    b = torch.from_numpy(rng.normal(0, 3, (4, 70000)).astype(np.float32)).cuda().to(torch.bfloat16)
    idx, _ = bs.argmax_rows(b)
    ref = b.float().cpu().numpy()
    for r in range(4):
        assert int(idx[r]) == orc.greedy(ref[r])


# ---- the reference's sampler known-answer tests through the mirrored API ----------------------
def test_sampler_api_known_answers():
    from opentail.stingray_b200 import Random, Sampler, SamplingParams

    assert Sampler.Greedy([1, 5, 3, 2]) == 1
    assert Sampler.Greedy([10, 1, 2, 3]) == 0
    assert Sampler.Greedy([1, 2, 3, 100]) == 3
    assert Sampler.Greedy([]) == 0
    assert Sampler.Sample([1, 5, 3, 2], SamplingParams(Temperature=0.0)) == 1
    rng = Random(42)
    # SamplerTests.cs:296-325
    assert Sampler.Sample([10, 9.8, 0], SamplingParams(TopK=1, PresencePenalty=1.0, PreviousTokens=[0]), rng) == 1
    assert Sampler.Sample([10, 9.8, 0], SamplingParams(TopK=1, FrequencyPenalty=0.6, PreviousTokens=[0, 0]), rng) == 1
    assert rng.draws == 2
    assert Sampler.Sample([10, 9.8], SamplingParams(Temperature=0.0, PresencePenalty=1.0, PreviousTokens=[0]), rng) == 1
    assert rng.draws == 2  # greedy consumes no draw
    # SamplerTests.cs:70-85, 257-294, 327-361
    seen = {Sampler.Sample(list(range(1, 11)), SamplingParams(TopK=2), rng) for _ in range(200)}
    assert seen <= {8, 9}
    seen = {Sampler.Sample([10, 8, 7, 1, 0], SamplingParams(TopK=2, RepetitionPenalty=4.0, PreviousTokens=[1]), rng)
            for _ in range(200)}
    assert 1 not in seen and seen <= {0, 2} and 2 in seen
    once = {Sampler.Sample([9, 8, 6.5, 1], SamplingParams(TopK=2, RepetitionPenalty=1.2, PreviousTokens=[1]), rng)
            for _ in range(200)}
    thrice = {Sampler.Sample([9, 8, 6.5, 1], SamplingParams(TopK=2, RepetitionPenalty=1.2, PreviousTokens=[1, 1, 1]), rng)
              for _ in range(200)}
    assert 1 in once and 1 not in thrice and 2 in thrice
    seen = {Sampler.Sample([2, NEG, 5, NEG, 1, 3], SamplingParams(TopK=5, TopP=0.95), rng) for _ in range(200)}
    assert seen <= {0, 2, 4, 5}
    assert 0 <= Sampler.Sample([NEG, NEG, NEG], SamplingParams(TopK=2, TopP=0.9), rng) <= 2
    seen = {Sampler.Sample([6, 3, 2.5, 0, 0, 0, 0, 0], SamplingParams(TopK=3, TopP=0.5), rng) for _ in range(100)}
    assert seen == {0}
    # logit bias, SamplerTests.cs:151-209
    seen = {Sampler.Sample([10, 1, 1, 1], SamplingParams(LogitBias={0: -100.0}), rng) for _ in range(100)}
    assert 0 not in seen
    seen = {Sampler.Sample([0, 0, 0, 0], SamplingParams(LogitBias={2: 100.0}), rng) for _ in range(100)}
    assert seen == {2}
    assert 0 <= Sampler.Sample([1, 2, 3], SamplingParams(LogitBias={999: 100.0, -1: 100.0}), rng) <= 2
    # distributions, SamplerTests.cs:365-401
    probs = np.zeros(4, np.float32)
    Sampler.BuildFilteredDistribution([1, 2, 3, 0], SamplingParams(), probs)
    e = np.exp(np.array([1, 2, 3, 0], np.float64) - 3)
    np.testing.assert_allclose(probs, e / e.sum(), atol=1e-5)
    Sampler.BuildFilteredDistribution([1, 9, 3, 2], SamplingParams(Temperature=0.0), probs)
    assert probs[1] == 1.0 and probs[0] + probs[2] + probs[3] == 0.0
    probs = np.zeros(5, np.float32)
    Sampler.BuildFilteredDistribution([5, 4, 3, 2, 1], SamplingParams(TopK=2), probs)
    assert probs[0] > 0 and probs[1] > 0 and probs[2] + probs[3] + probs[4] == 0 and abs(probs.sum() - 1) < 1e-5
    with pytest.raises(ValueError):
        Sampler.BuildFilteredDistribution([1, 2, 3], SamplingParams(), np.zeros(4, np.float32))


# ---- randomised parity against the oracle -----------------------------------------------------------
@pytest.mark.parametrize("vocab", [1, 2, 3, 31, 32, 33, 255, 256, 257, 1000, 4097, 20000])
def test_small_vocab_all_paths(bs, vocab):
    rng = np.random.default_rng(vocab)
    rows = 24
    logits = rng.normal(0, 3, (rows, vocab)).astype(np.float32)
    p = _params(rows)
    p["temperature"] = rng.choice(np.array([0.0, 0.5, 1.0, 1.3], np.float32), rows)
    p["top_k"] = rng.choice(np.array([0, 1, 5, 40, 900]), rows)
    p["top_p"] = rng.choice(np.array([1.0, 0.9, 0.5], np.float32), rows)
    p["min_p"] = rng.choice(np.array([0.0, 0.05], np.float32), rows)
    p["repetition_penalty"] = rng.choice(np.array([1.0, 1.1, 1.3], np.float32), rows)
    p["presence_penalty"] = rng.choice(np.array([0.0, 0.3], np.float32), rows)
    p["frequency_penalty"] = rng.choice(np.array([0.0, 0.5], np.float32), rows)
    p["repeat_last_n"] = rng.choice(np.array([0, 4, 64]), rows)
    hist = [rng.integers(-2, vocab + 2, rng.integers(0, 40)) for _ in range(rows)]
    from opentail.stingray_b200 import workloads as W

    w = _wl(logits, p, W.uniforms24(rng, rows), hist)
    gpu = parity.run_gpu(bs, w, want_topk=int(min(p["top_k"].max(), 1024)) or 1)
    stats = parity.compare(w, gpu)
    assert stats["boundary_draws"] <= 1


def test_ties_duplicates_and_neg_inf(bs):
    rng = np.random.default_rng(7)
    rows, vocab = 16, 5000
    logits = rng.integers(-3, 4, (rows, vocab)).astype(np.float32)  # heavy ties
    logits[0, :] = 2.0                                              # constant row
    logits[1, :] = NEG                                              # fully masked row, top-k path
    logits[2, :] = NEG                                              # fully masked row, full path
    logits[3, 100:] = NEG
    p = _params(rows, temperature=0.9, top_k=50, top_p=0.95)
    p["top_k"][2] = 0
    p["top_k"][8:] = 0
    hist = [rng.integers(0, vocab, 30) for _ in range(rows)]
    p["repetition_penalty"] = 1.2
    from opentail.stingray_b200 import workloads as W

    w = _wl(logits, p, W.uniforms24(rng, rows), hist)
    gpu = parity.run_gpu(bs, w, want_topk=50)
    stats = parity.compare(w, gpu)
    assert gpu["tokens"][1] == 0 and (gpu["flags"][1] & 7) == 4
    assert stats["mismatch"] == stats["boundary_draws"]


def test_promoting_penalties_two_stage_selection(bs):
    """Penalties that PROMOTE (repetition < 1, negative presence): the reference selects the raw
    top-(k + history) first and penalises only those; the result differs from 'penalise then
    top-k', and the library must follow the reference."""
    rng = np.random.default_rng(11)
    rows, vocab = 12, 8000
    logits = rng.normal(0, 2, (rows, vocab)).astype(np.float32)
    p = _params(rows, temperature=0.8, top_k=8, top_p=0.9, repetition_penalty=0.5, presence_penalty=-2.0,
                repeat_last_n=0)
    hist = [rng.integers(0, vocab, 16) for _ in range(rows)]
    from opentail.stingray_b200 import workloads as W

    w = _wl(logits, p, W.uniforms24(rng, rows), hist)
    gpu = parity.run_gpu(bs, w, want_topk=8)
    parity.compare(w, gpu)


def test_sorted_and_drifting_rows_selection_retry(bs):
    """Rows whose first elements are not representative of the rest (descending, ascending, a step):
    the streaming selection guesses its threshold from the first sub-tile and must notice a guess
    that keeps too few candidates."""
    rng = np.random.default_rng(21)
    vocab = 151936
    base = rng.normal(0, 2.5, (6, vocab)).astype(np.float32)
    logits = base.copy()
    logits[0] = np.sort(base[0])[::-1]                      # largest values first
    logits[1] = np.sort(base[1])                            # largest values last
    logits[2, :8192] += 6.0                                 # a block of large values at the start
    logits[3, 8192:] += 6.0                                 # ... everywhere but the start
    logits[4] = np.round(base[4])                           # heavy ties
    logits[4, :4096] = 9.0                                  # the whole first sub-tile is one tied maximum
    p = _params(6, temperature=0.9, top_k=64, top_p=0.95, repetition_penalty=1.1, frequency_penalty=0.2)
    hist = [rng.integers(0, vocab, 200) for _ in range(6)]
    from opentail.stingray_b200 import workloads as W

    w = _wl(logits, p, W.uniforms24(rng, 6), hist)
    gpu = parity.run_gpu(bs, w, want_topk=64)
    stats = parity.compare(w, gpu)
    assert stats["mismatch"] == stats["boundary_draws"]
    # the same rows as many-row batch (one chunk per row: long ranges)
    from opentail.stingray_b200 import BatchSampler

    big = np.tile(logits, (50, 1))
    pb = np.tile(p, 50)
    wb = _wl(big, pb, W.uniforms24(rng, 300), [hist[i % 6] for i in range(300)])
    bs2 = BatchSampler(max_rows=300, max_vocab=vocab, max_history=256, max_top_k=64)
    gb = parity.run_gpu(bs2, wb, want_topk=64)
    bs2.close()
    for r in range(300):
        assert np.array_equal(gb["topk_ids"][r, :64], gpu["topk_ids"][r % 6, :64]), r


def test_logit_bias_rows_against_oracle(bs):
    """Rows with logit bias take the full-vocabulary path, where top-k is ApplyTopK + Normalize
    (Sampler.cs:41-95): bias entries (duplicates, out-of-range ids, promoting and demoting values),
    histories, top-k / min-p / top-p on and off, on a full-size vocabulary."""
    import torch

    rng = np.random.default_rng(31)
    rows, vocab = 24, 151936
    logits = rng.normal(0, 2.5, (rows, vocab)).astype(np.float32)
    p = _params(rows, temperature=0.9, top_p=0.92)
    p["temperature"] = rng.uniform(0.4, 1.3, rows).astype(np.float32)
    p["top_k"] = rng.choice([0, 0, 30, 200], rows)
    p["min_p"] = rng.choice([0.0, 0.0, 0.02], rows).astype(np.float32)
    p["top_p"] = rng.choice([1.0, 0.9, 0.97], rows).astype(np.float32)
    p["repetition_penalty"] = rng.choice([1.0, 1.15], rows).astype(np.float32)
    p["frequency_penalty"] = rng.choice([0.0, 0.4], rows).astype(np.float32)
    hist = [rng.integers(0, vocab, 100) for _ in range(rows)]
    bias = []
    for r in range(rows):
        n = int(rng.integers(3, 40))
        ids = rng.integers(-5, vocab + 5, n)
        top = np.argsort(logits[r])[-3:]
        ids[-3:] = top                                           # push the best tokens around
        ids = np.unique(ids)                                     # LogitBias is a dictionary: distinct keys
        vals = rng.choice([-100.0, -3.0, 2.5, 8.0], ids.size).astype(np.float32)
        bias.append((ids.astype(np.int32), vals))
    bi = np.concatenate([b[0] for b in bias])
    bv = np.concatenate([b[1] for b in bias])
    bo = np.concatenate([[0], np.cumsum([len(b[0]) for b in bias])]).astype(np.int32)
    from opentail.stingray_b200 import workloads as W

    u = W.uniforms24(rng, rows)
    w = _wl(logits, p, u, hist)
    out = bs.sample_rows(torch.from_numpy(logits).cuda(), p, history_ids=torch.from_numpy(w.history_ids).cuda(),
                         history_offsets=w.history_offsets, bias=(torch.from_numpy(bi).cuda(), torch.from_numpy(bv).cuda(), bo),
                         uniforms=torch.from_numpy(u).cuda(), want_probs=True, want_flags=True)
    tok = out["tokens"].cpu().numpy()
    prob = out["probs"].cpu().numpy()
    flags = out["flags"].cpu().numpy().view(np.uint32)
    mismatch = 0
    for r in range(rows):
        op = orc.OrcParams(*[p[r][n].item() for n in p.dtype.names])
        ids, vals = bias[r]
        res = orc.sample_bias_arrays(logits[r], op, float(u[r]), hist[r], ids, vals)
        assert (flags[r] & 7) == 3
        if tok[r] != res.token:
            assert float(res.trace.margin) <= parity.BOUNDARY, (r, tok[r], res.token, res.trace.margin)
            mismatch += 1
        else:
            np.testing.assert_allclose(prob[r], res.trace.prob, rtol=2e-5)
    assert mismatch <= 1


def test_top_p_never_reached_after_min_p(bs):
    """min-p can remove so much mass that the running sum of ApplyTopP never reaches top_p; nothing
    is cut then (Sampler.cs:536-549).  Also the wide-nucleus case (keys outside shared memory)."""
    from opentail.stingray_b200 import workloads as W

    rng = np.random.default_rng(41)
    for vocab, sigma, temp, top_p, min_p in ((200003, 6.0, 0.7, 0.5, 0.2), (32000, 2.0, 1.5, 0.99, 0.01),
                                              (151936, 1.0, 1.5, 0.9999, 0.001), (262144, 2.0, 1.5, 0.9999, 0.0),
                                              (200003, 3.5, 1.5, 0.9999, 0.0)):
        rows = 6
        logits = rng.normal(0, sigma, (rows, vocab)).astype(np.float32)
        p = _params(rows, temperature=temp, top_p=top_p, min_p=min_p, repetition_penalty=1.1, presence_penalty=-0.5,
                    repeat_last_n=0)
        hist = [rng.integers(0, vocab, 300) for _ in range(rows)]
        w = _wl(logits, p, W.uniforms24(rng, rows), hist)
        first = parity.run_gpu(bs, w)
        stats = parity.compare(w, first)
        assert stats["mismatch"] == 0
        again = parity.run_gpu(bs, w)
        assert np.array_equal(first["tokens"], again["tokens"])


def test_config1_single_row_and_greedy(bs):
    from opentail.stingray_b200 import workloads as W

    w = W.config1()
    gpu = parity.run_gpu(bs, w, want_topk=40)
    stats = parity.compare(w, gpu)
    assert stats["paths"] == {2: 1} and stats["mismatch"] == 0
    g = W.config1(greedy=True)
    gpu = parity.run_gpu(bs, g)
    parity.compare(g, gpu)
    assert (gpu["flags"][0] & 7) == 1  # greedy with penalties


def test_config2_server_decode_slice(bs):
    from opentail.stingray_b200 import workloads as W

    w = W.config2(rows=48)
    gpu = parity.run_gpu(bs, w, want_topk=100)
    stats = parity.compare(w, gpu)
    assert stats["paths"].get(2, 0) > 0 and stats["paths"].get(3, 0) > 0
    assert stats["boundary_draws"] <= 1, stats


def test_config3_grammar_mask_slice(bs):
    from opentail.stingray_b200 import workloads as W

    w = W.config3(rows=12)
    gpu = parity.run_gpu(bs, w)
    stats = parity.compare(w, gpu)
    allowed = np.unpackbits(w.mask.view(np.uint8), axis=1, bitorder="little")
    for r in range(w.rows):
        assert allowed[r, gpu["tokens"][r]] == 1, "a masked token was sampled"
    assert stats["boundary_draws"] <= 1, stats


def test_config5_slice_and_chunk_merge(bs):
    from opentail.stingray_b200 import workloads as W

    w = W.config5(rows=6)  # few rows: every row is split into many chunks and merged
    gpu = parity.run_gpu(bs, w, want_topk=50)
    stats = parity.compare(w, gpu)
    assert stats["mismatch"] == 0


def test_determinism_and_host_arrays(bs):
    from opentail.stingray_b200 import workloads as W

    w = W.config2(rows=8, vocab=30000)
    a = parity.run_gpu(bs, w, want_topk=100)
    b = parity.run_gpu(bs, w, want_topk=100)
    for k in a:
        assert np.array_equal(a[k], b[k]), k
    host = bs.sample_rows(w.logits, w.params, history_ids=w.history_ids, history_offsets=w.history_offsets,
                          uniforms=w.uniforms, want_probs=True)
    assert np.array_equal(host["tokens"], a["tokens"])


def test_distribution_matches_oracle(bs):
    import torch

    rng = np.random.default_rng(21)
    rows, vocab = 10, 30000
    logits = rng.normal(0, 2.5, (rows, vocab)).astype(np.float32)
    p = _params(rows)
    p["temperature"] = rng.uniform(0.4, 1.2, rows).astype(np.float32)
    p["top_k"] = [0, 0, 40, 0, 200, 0, 0, 3, 0, 0]
    p["top_p"] = [1.0, 0.9, 0.9, 0.5, 1.0, 0.95, 0.99, 1.0, 0.8, 0.9]
    p["min_p"] = [0.0, 0.0, 0.0, 0.02, 0.0, 0.05, 0.0, 0.0, 0.0, 0.0]
    p["temperature"][9] = 0.0
    got = bs.build_distribution(torch.from_numpy(logits).cuda(), p).cpu().numpy()
    for r in range(rows):
        op = orc.OrcParams(*[p[r][n].item() for n in p.dtype.names])
        want, tie = orc.build_filtered_distribution(logits[r], op)
        assert np.array_equal(got[r] > 0, want > 0), f"row {r}: support differs"
        np.testing.assert_allclose(got[r], want, rtol=1e-5, atol=1e-30, err_msg=f"row {r}")


def test_capacity_and_argument_errors(bs):
    import torch
    from opentail.stingray_b200 import StingrayError

    x = torch.zeros((2, 300000), device="cuda")
    with pytest.raises(StingrayError) as e:
        bs.sample_rows(x, _params(2), uniforms=np.array([0.5, 0.5], np.float32))
    assert e.value.code == 3
    x = torch.zeros((2, 10000), device="cuda")
    with pytest.raises(StingrayError) as e:
        bs.sample_rows(x, _params(2, top_k=5000), uniforms=np.array([0.5, 0.5], np.float32))
    assert e.value.code == 3
