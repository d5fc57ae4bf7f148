"""Pins the CPU oracle against the reference's own known-answer tests.

Each test restates one test of the reference's suites on the same literals:
  SamplerTests            tests/OpenTail.Stingray.Tests.ForwardPass.Fast/SamplerTests.cs
  SpeculativeSamplingTests   .../SpeculativeSamplingTests.cs
  CudaGpuArgmaxParityTests   tests/OpenTail.Stingray.Tests.Cuda/CudaGpuArgmaxParityTests.cs
Where the reference draws from System.Random (which cannot be regenerated without .NET), the
same property is checked over a dense grid of uniforms instead of a random stream.
"""
import math

import numpy as np
import pytest

from oracle import oracle as orc

NEG = -math.inf
GRID = [(j + 0.5) / 4096 for j in range(4096)]


def reach(logits, p, history=None, bias=None, grid=GRID):
    return {orc.sample(logits, p, u, history=history, bias=bias).token for u in grid}


# ---- SamplerTests.cs:7-34 ------------------------------------------------------------------
def test_greedy_returns_argmax():
    assert orc.greedy([1, 5, 3, 2]) == 1
    assert orc.greedy([10, 1, 2, 3]) == 0
    assert orc.greedy([1, 2, 3, 100]) == 3


def test_temperature_zero_is_greedy():
    assert orc.sample([1, 5, 3, 2], orc.make_params(temperature=0.0)).token == 1


# ---- SamplerTests.cs:36-147 (statistical tests restated over the uniform grid) ---------------
def test_very_low_temperature_peaks_at_max():
    picks = [orc.sample([1, 10, 2, 3], orc.make_params(temperature=0.001), u).token for u in GRID]
    assert sum(t == 1 for t in picks) >= 0.99 * len(GRID)


def test_high_temperature_more_uniform():
    picks = [orc.sample([0, 0, 0, 10], orc.make_params(temperature=100.0), u).token for u in GRID]
    for i in range(4):
        assert 0.15 * len(GRID) <= sum(t == i for t in picks) <= 0.35 * len(GRID)


def test_top_k_restricts_to_k_tokens():
    assert reach(list(range(1, 11)), orc.make_params(top_k=2)) <= {8, 9}


def test_top_p_restricts_to_nucleus():
    picks = [orc.sample([0] * 9 + [20], orc.make_params(top_p=0.5), u).token for u in GRID]
    assert sum(t == 9 for t in picks) >= 0.95 * len(GRID)


def test_min_p_filters_low_prob_tokens():
    r = reach([0] * 9 + [50], orc.make_params(min_p=0.1))
    assert 9 in r and len(r) <= 2


def test_uniform_logits_all_tokens_sampled():
    assert reach([0, 0, 0, 0], orc.make_params()) == {0, 1, 2, 3}


# ---- SamplerTests.cs:151-209 logit bias ------------------------------------------------------
def test_logit_bias():
    assert 0 not in reach([10, 1, 1, 1], orc.make_params(), bias={0: -100.0})
    assert reach([0, 0, 0, 0], orc.make_params(), bias={2: 100.0}) == {2}
    r = reach([1, 2, 3], orc.make_params(), bias={999: 100.0, -1: 100.0})
    assert r <= {0, 1, 2}


# ---- SamplerTests.cs:234-255 fast path == forced slow path (reachable set) ------------------
@pytest.mark.parametrize("seed", [1, 7, 99])
def test_fast_path_matches_slow_path_reachable_set(seed):
    rng = np.random.default_rng(seed)
    logits = (rng.random(96) * 12 - 6).astype(np.float32)
    p = orc.make_params(temperature=0.8, top_k=16, top_p=0.9, min_p=0.02, repetition_penalty=1.3)
    hist = [3, 3, 10, 25]
    fast = reach(logits, p, history=hist)
    slow = reach(logits, p, history=hist, bias={-1: 0.0})
    assert orc.sample(logits, p, 0.5, history=hist).trace.path == 2
    assert orc.sample(logits, p, 0.5, history=hist, bias={-1: 0.0}).trace.path == 3
    assert fast == slow


# ---- SamplerTests.cs:257-294 penalties demote ----------------------------------------------
def test_penalty_demotes_out_of_top_k():
    p = orc.make_params(top_k=2, repetition_penalty=4.0)
    r = reach([10, 8, 7, 1, 0], p, history=[1])
    assert 1 not in r and r <= {0, 2} and 2 in r


def test_duplicate_occurrences_compound():
    logits = [9, 8, 6.5, 1]
    p = orc.make_params(top_k=2, repetition_penalty=1.2)
    once = reach(logits, p, history=[1])
    thrice = reach(logits, p, history=[1, 1, 1])
    assert 1 in once
    assert 1 not in thrice and 2 in thrice


# ---- SamplerTests.cs:296-325 presence / frequency -------------------------------------------
def test_presence_and_frequency_penalties():
    logits = [10, 9.8, 0]
    for u in (0.01, 0.5, 0.99):
        assert orc.sample(logits, orc.make_params(top_k=1, presence_penalty=1.0), u,
                          history=[0]).token == 1
        assert orc.sample(logits, orc.make_params(top_k=1, frequency_penalty=0.6), u,
                          history=[0, 0]).token == 1


def test_greedy_honours_presence_penalty():
    p = orc.make_params(temperature=0.0, presence_penalty=1.0)
    r = orc.sample([10, 9.8], p, history=[0])
    assert r.token == 1 and r.trace.path == 1


# ---- SamplerTests.cs:327-361 -inf handling, top-k then top-p -----------------------------------
def test_neg_inf_logits_never_sampled():
    logits = [2, NEG, 5, NEG, 1, 3]
    r = reach(logits, orc.make_params(top_k=5, top_p=0.95))
    assert r <= {0, 2, 4, 5}


def test_all_neg_inf_falls_back_to_valid_token():
    r = orc.sample([NEG, NEG, NEG], orc.make_params(top_k=2, top_p=0.9), 0.3)
    assert 0 <= r.token <= 2 and r.trace.path == 4


def test_top_k_then_top_p_nucleus_after_top_k():
    r = reach([6, 3, 2.5, 0, 0, 0, 0, 0], orc.make_params(top_k=3, top_p=0.5))
    assert r == {0}


# ---- SamplerTests.cs:365-413 distribution helpers ---------------------------------------------
def test_build_filtered_distribution_matches_softmax():
    logits = [1, 2, 3, 0]
    probs, _ = orc.build_filtered_distribution(logits, orc.make_params())
    e = np.exp(np.array(logits, np.float64) - 3.0)
    np.testing.assert_allclose(probs, e / e.sum(), atol=1e-5)
    assert abs(float(probs.sum()) - 1.0) < 1e-5


def test_build_filtered_distribution_temp_zero_one_hot():
    probs, _ = orc.build_filtered_distribution([1, 9, 3, 2], orc.make_params(temperature=0.0))
    assert probs[1] == 1.0 and probs[0] + probs[2] + probs[3] == 0.0


def test_build_filtered_distribution_top_k():
    probs, _ = orc.build_filtered_distribution([5, 4, 3, 2, 1], orc.make_params(top_k=2))
    assert probs[0] > 0 and probs[1] > 0
    assert probs[2] + probs[3] + probs[4] == 0.0
    assert abs(float(probs.sum()) - 1.0) < 1e-5


def test_sample_with_distribution():
    for u in (0.02, 0.5, 0.97):
        tok, probs, _ = orc.sample_with_distribution([0, 12, 0, 0], orc.make_params(temperature=0.1), u)
        assert tok == 1 and probs[1] > 0.99 and abs(float(probs.sum()) - 1.0) < 1e-5


# ---- SamplerTests.cs:415-442 residual -----------------------------------------------------------
def test_resample_residual_concentrated():
    for u in GRID[::16]:
        tok, used, _ = orc.resample_residual([0, 0.5, 0.5, 0], [0, 1.0, 0.0, 0], u)
        assert tok == 2 and used == 1


def test_resample_residual_empty_falls_back_to_p():
    seen = set()
    for u in GRID[::16]:
        tok, used, _ = orc.resample_residual([0.25] * 4, [0.25] * 4, u)
        assert 0 <= tok <= 3
        seen.add(tok)
    assert seen == {0, 1, 2, 3}


def test_resample_residual_mismatched_lengths_throws():
    with pytest.raises(ValueError):
        orc.resample_residual([0.0] * 4, [0.0] * 3, 0.5)


# ---- SpeculativeSamplingTests.cs:21-50 distribution preservation --------------------------------
P_TARGET = [0.2, 2.5, 0.1, 1.0, 0.3, 1.8, 0.0, 0.5]
Q_DRAFT = [2.0, 0.1, 1.5, 0.2, 1.0, 0.0, 2.2, 0.3]


def test_sampled_spec_preserves_target_distribution():
    """One draft position per step, every uniform seeded: the emitted-token histogram of the
    accept/residual rule must match softmax(PTarget) within 0.02 and the acceptance rate must be
    strictly inside (0.01, 0.99) - the invariant SampledSpec_PreservesTargetDistribution checks."""
    rng = np.random.default_rng(12345)
    p = orc.make_params()
    n = 20000
    counts = np.zeros(8)
    accepted = 0
    target = np.array([P_TARGET, P_TARGET], np.float32)
    draft = np.array([Q_DRAFT], np.float32)
    for _ in range(n):
        u = rng.random(4)
        x, _, _ = orc.sample_with_distribution(Q_DRAFT, p, u[0])
        acc, corr, _, _ = orc.spec_step_sampled(target, draft, [x], p, [u[1]], [u[2], u[3]])
        accepted += acc
        # the emitted token at this slot is the draft when accepted, else the correction
        counts[x if acc == 1 else corr] += 1
    e = np.exp(np.array(P_TARGET) - max(P_TARGET))
    expected = e / e.sum()
    assert np.abs(counts / n - expected).max() < 0.02
    assert 0.01 < accepted / n < 0.99


def test_sampled_spec_same_uniforms_deterministic():
    p = orc.make_params()
    target = np.array([P_TARGET] * 4, np.float32)
    draft = np.array([Q_DRAFT] * 3, np.float32)
    a = orc.spec_step_sampled(target, draft, [6, 0, 2], p, [0.3, 0.6, 0.1], [0.7, 0.2])
    b = orc.spec_step_sampled(target, draft, [6, 0, 2], p, [0.3, 0.6, 0.1], [0.7, 0.2])
    assert a[0] == b[0] and a[1] == b[1]


def test_spec_temp_zero_routes_to_greedy():
    # SamplingCtor_TempZero_RoutesToGreedy: greedy emits argmax(p) everywhere; the draft's
    # argmax (token 6) never matches it.
    rows = np.array([P_TARGET] * 3, np.float32)
    assert orc.greedy(P_TARGET) == 1
    assert orc.spec_greedy_accept(rows, [6, 6, 6]) == 0
    assert orc.spec_greedy_accept(rows, [1, 1, 6]) == 2


def test_pmin_looser_accept_produces_valid_tokens():
    p = orc.make_params()
    target = np.array([P_TARGET] * 4, np.float32)
    draft = np.array([Q_DRAFT] * 3, np.float32)
    for u in GRID[::64]:
        acc, corr, _, _ = orc.spec_step_sampled(target, draft, [6, 0, 2], p, [0.5] * 3, [u, 0.5],
                                                mode=1, p_min=0.05)
        assert 0 <= acc <= 3 and 0 <= corr < 8


# ---- CudaGpuArgmaxParityTests.cs:57-176 -----------------------------------------------------------
def _cpu_argmax(a):
    idx, best = 0, a[0]
    for i in range(1, len(a)):
        if a[i] > best:
            best, idx = a[i], i
    return idx


@pytest.mark.parametrize("n", [1, 2, 3, 255, 256, 257, 1000, 65536, 152064, 262144])
def test_argmax_sizes_and_positions(n):
    rng = np.random.default_rng(1234 + n)
    a = (rng.random(n) * 20 - 10).astype(np.float32)
    assert orc.greedy(a) == int(np.argmax(a))
    for pos in (0, n // 2, n - 1):
        b = a.copy()
        b[pos] = 1000.0 + pos
        assert orc.greedy(b) == pos


def test_argmax_ties_and_constant_rows():
    a = np.full(5000, -1.0, np.float32)
    a[700] = 5.0
    a[300] = 5.0
    assert orc.greedy(a) == 300
    assert orc.greedy(np.full(8192, 3.5, np.float32)) == 0
    rng = np.random.default_rng(99)
    neg = (-rng.random(4096) * 50 - 1).astype(np.float32)
    assert orc.greedy(neg) == _cpu_argmax(neg)


# ---- mask semantics: ITokenConstraint.cs:31-43, AndTokenConstraintTests.cs:132-216 -------------
def _bits(ids, n):
    m = np.zeros((n + 31) // 32, np.uint32)
    for i in ids:
        m[i >> 5] |= np.uint32(1 << (i & 31))
    return m


def test_mask_sets_forbidden_to_neg_inf_and_keeps_allowed():
    logits = np.arange(40, dtype=np.float32)
    out = orc.apply_mask(logits, _bits([3, 33], 40))
    assert out[3] == 3 and out[33] == 33
    assert np.isneginf(np.delete(out, [3, 33])).all()
    # ConstrainedChoiceSamplingTests.cs:41-64: the illegal highest-logit token is masked
    assert orc.greedy(out) == 33


def test_and_masks_intersection_and_dead_states():
    n = 40
    out, masking = orc.and_masks([_bits([1, 2, 35], n), _bits([2, 35, 36], n)], n)
    assert masking and set(np.flatnonzero(np.unpackbits(out.view(np.uint8), bitorder="little")[:n])) == {2, 35}
    # empty intersection => unmasked (AndTokenConstraint.cs:80-85)
    out, masking = orc.and_masks([_bits([1], n), _bits([2], n)], n)
    assert not masking and (out == 0xFFFFFFFF).all()
    # a dead inner (no legal token) is skipped (AndTokenConstraint.cs:71)
    out, masking = orc.and_masks([_bits([], n), _bits([5], n)], n)
    assert masking and out[0] == 1 << 5


# ---- MTP p-min rule: MtpDecoder.cs:562-596 (no reference test exercises pMin < 1) -------------
def test_mtp_accept_rule():
    logits = np.array([0.0, 2.0, 1.0], np.float32)
    assert orc.mtp_accept(logits, 1, 1.0) == (True, 0.0)
    assert orc.mtp_accept(logits, 2, 1.0) == (False, 0.0)
    ok, pr = orc.mtp_accept(logits, 2, 0.2)
    e = np.exp(np.array([-2.0, 0.0, -1.0]))
    assert ok and abs(pr - e[2] / e.sum()) < 1e-7
    assert orc.mtp_accept(logits, 2, 0.0)[0] is False  # pMin <= 0 is treated as 1


# ---- A3 vs A4 penalty forms ----------------------------------------------------------------------
def test_slow_penalty_compounds_by_repeated_division():
    p = orc.make_params(repetition_penalty=1.2, repeat_last_n=0, presence_penalty=0.25,
                        frequency_penalty=0.5)
    out = orc.apply_history_penalties([8.0, -2.0, 1.0], p, [0, 0, 0, 1, 7, -3])
    x = np.float32(8.0)
    for _ in range(3):
        x = np.float32(x / np.float32(1.2))
    x = np.float32(x - np.float32(np.float32(0.25) + np.float32(np.float32(0.5) * np.float32(3))))
    assert out[0] == x
    y = np.float32(np.float32(-2.0) * np.float32(1.2))
    y = np.float32(y - np.float32(np.float32(0.25) + np.float32(0.5)))
    assert out[1] == y and out[2] == 1.0


def test_repeat_window_limits_repetition_but_not_frequency():
    p = orc.make_params(repetition_penalty=2.0, repeat_last_n=2, frequency_penalty=1.0)
    out = orc.apply_history_penalties([8.0, 8.0], p, [0, 0, 1, 1])
    assert out[0] == 8.0 - 2.0 and out[1] == 8.0 / 4 - 2.0
