"""GPU parity tests of speculative verification, the MTP accept rule and the vocabulary-sharded mode."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import parity

pytestmark = pytest.mark.gpu


def _params(rows, **kw):
    from opentail.stingray_b200 import workloads as W

    return W._params(rows, **kw)


def _oracle_draw(params_row):
    def draw(draft, u):
        n_seq, L, _ = draft.shape
        toks = np.zeros((n_seq, L), np.int32)
        p = orc.OrcParams(*[params_row[n].item() for n in params_row.dtype.names])
        for s in range(n_seq):
            for i in range(L):
                toks[s, i], _, _ = orc.sample_with_distribution(draft[s, i], p, float(u[s, i]))
        return toks
    return draw


def _check_spec(w, mode=0, p_min=1.0, boundary_budget=1):
    import torch
    from opentail.stingray_b200 import BatchSampler

    n_seq, lp1, vocab = w.target.shape
    L = lp1 - 1
    bs = BatchSampler(max_rows=n_seq * lp1, max_vocab=vocab, max_history=1, max_top_k=64, max_spec_draft=L)
    try:
        out = bs.spec_verify(torch.from_numpy(w.target).cuda(), torch.from_numpy(w.draft).cuda(), w.draft_tokens,
                             w.params, w.uniforms, mode=mode, p_min=p_min, want_probs=True)
        torch.cuda.synchronize()
        acc, corr, ap = out["accepted"].cpu().numpy(), out["correction"].cpu().numpy(), out["accept_probs"].cpu().numpy()
    finally:
        bs.close()
    boundary = 0
    for s in range(n_seq):
        p = orc.OrcParams(*[w.params[s][n].item() for n in w.params.dtype.names])
        if p.temperature <= 0:
            want_acc = orc.spec_greedy_accept(w.target[s, :L], w.draft_tokens[s])
            assert acc[s] == want_acc
            assert corr[s] == orc.greedy(w.target[s, want_acc])
            continue
        want_acc, want_corr, want_ap, tr = orc.spec_step_sampled(
            w.target[s], w.draft[s], w.draft_tokens[s], p, w.uniforms[s, :L], w.uniforms[s, L:], mode=mode, p_min=p_min)
        tested = min(want_acc + 1, L)
        np.testing.assert_allclose(ap[s, :tested], want_ap[:tested], rtol=2e-5, atol=1e-30, err_msg=f"seq {s}")
        if acc[s] != want_acc:
            # an accept test within tolerance of its uniform may flip
            i = min(acc[s], want_acc)
            assert abs(float(w.uniforms[s, i]) - float(want_ap[i])) <= 2e-5 * max(float(want_ap[i]), 1e-30), f"seq {s}"
            boundary += 1
            continue
        if corr[s] != want_corr:
            assert tr.margin <= parity.BOUNDARY, f"seq {s}: correction {corr[s]} != {want_corr}, margin {tr.margin}"
            boundary += 1
    assert boundary <= boundary_budget
    return acc, corr


def test_spec_verify_config4_slice():
    from opentail.stingray_b200 import workloads as W

    p = _params(1)
    w = W.config4(n_seq=6, n_draft=4, vocab=20000, draw_tokens=_oracle_draw(p[0]))
    acc, _ = _check_spec(w)
    assert acc.min() >= 0 and acc.max() <= 4


def test_spec_verify_full_vocab_and_filters():
    from opentail.stingray_b200 import workloads as W

    p = _params(1)
    w = W.config4(n_seq=3, n_draft=3, draw_tokens=_oracle_draw(p[0]))
    _check_spec(w)
    # the same with top-k / top-p / temperature on both distributions (BuildFilteredDistribution)
    q = _params(4, temperature=0.8, top_k=50, top_p=0.9)
    w = W.config4(n_seq=4, n_draft=3, vocab=30000, seed=13, draw_tokens=_oracle_draw(q[0]))
    w.params = q
    _check_spec(w)


def test_spec_verify_looser_rule_and_greedy():
    from opentail.stingray_b200 import workloads as W

    p = _params(1)
    w = W.config4(n_seq=5, n_draft=4, vocab=12000, seed=5, draw_tokens=_oracle_draw(p[0]))
    _check_spec(w, mode=1, p_min=0.0005)
    g = W.config4(n_seq=4, n_draft=4, vocab=12000, seed=6)
    g.params = _params(4, temperature=0.0)
    # make some drafts match the target argmax so that greedy accepts a prefix
    for s in range(4):
        for i in range(4):
            am = int(np.argmax(g.target[s, i]))
            g.draft_tokens[s, i] = am if i < s else (am + 1) % 12000
    acc, _ = _check_spec(g)
    assert list(acc) == [0, 1, 2, 3]


def test_spec_reference_literals():
    """SpeculativeSamplingTests.cs:21-50 literals: 8-token vocabulary, fixed target and draft rows."""
    import torch
    from opentail.stingray_b200 import BatchSampler

    P = np.array([0.2, 2.5, 0.1, 1.0, 0.3, 1.8, 0.0, 0.5], np.float32)
    Q = np.array([2.0, 0.1, 1.5, 0.2, 1.0, 0.0, 2.2, 0.3], np.float32)
    rng = np.random.default_rng(12345)
    n_seq, L = 64, 3
    target = np.tile(P, (n_seq, L + 1, 1))
    draft = np.tile(Q, (n_seq, L, 1))
    par = _params(n_seq)
    op = orc.make_params()
    toks = np.array([[orc.sample_with_distribution(Q, op, rng.random())[0] for _ in range(L)] for _ in range(n_seq)], np.int32)
    uni = rng.random((n_seq, L + 2))
    bs = BatchSampler(max_rows=n_seq * (L + 1), max_vocab=8, max_history=1, max_top_k=8, max_spec_draft=L)
    out = bs.spec_verify(torch.from_numpy(target).cuda(), torch.from_numpy(draft).cuda(), toks, par, uni)
    acc, corr = out["accepted"].cpu().numpy(), out["correction"].cpu().numpy()
    bs.close()
    for s in range(n_seq):
        a, c, _, _ = orc.spec_step_sampled(target[s], draft[s], toks[s], op, uni[s, :L], uni[s, L:])
        assert (acc[s], corr[s]) == (a, c)
    assert 0 < acc.mean() < L


def test_mtp_accept_rule():
    import torch
    from opentail.stingray_b200 import BatchSampler

    rng = np.random.default_rng(3)
    rows, vocab = 12, 50000
    logits = rng.normal(0, 3, (rows, vocab)).astype(np.float32)
    draft = rng.integers(0, vocab, rows).astype(np.int32)
    draft[:4] = logits[:4].argmax(axis=1)
    order = np.argsort(-logits[4:8], axis=1)
    draft[4:8] = order[:, 1]  # runner-up: sizeable probability
    bs = BatchSampler(max_rows=rows, max_vocab=vocab)
    try:
        for p_min in (1.0, 0.05, 0.0):
            acc, am, pr = bs.mtp_accept(torch.from_numpy(logits).cuda(), torch.from_numpy(draft).cuda(), p_min)
            acc, am, pr = acc.cpu().numpy(), am.cpu().numpy(), pr.cpu().numpy()
            for r in range(rows):
                ok, want_pr = orc.mtp_accept(logits[r], int(draft[r]), p_min)
                assert am[r] == orc.greedy(logits[r])
                assert bool(acc[r]) == ok, (r, p_min)
                np.testing.assert_allclose(pr[r], want_pr, rtol=1e-6, atol=1e-30)
    finally:
        bs.close()


@pytest.mark.parametrize("n_ranks", [2, 8])
def test_vocab_sharded_equals_unsharded(n_ranks):
    """Every rank selects over its vocabulary slice, the candidate lists are exchanged (here by
    device copies standing in for the NCCL all-gather) and merged; tokens, candidates and
    probabilities must equal the unsharded run's and the oracle's."""
    import torch
    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import workloads as W

    w = W.config5(rows=24, vocab=64000)
    w.params["temperature"][:4] = 0.0           # plain greedy rows ride along
    w.params["repetition_penalty"][:4] = 1.0
    mk = lambda: BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=256, max_top_k=64)
    full = mk()
    ref = parity.run_gpu(full, w, want_topk=50)
    parity.compare(w, ref)
    width = w.vocab // n_ranks
    ranks = [mk() for _ in range(n_ranks)]
    hist = torch.from_numpy(w.history_ids).cuda()
    uni = torch.from_numpy(w.uniforms).cuda()
    try:
        for r, bs in enumerate(ranks):
            sl = torch.from_numpy(np.ascontiguousarray(w.logits[:, r * width:(r + 1) * width])).cuda()
            bs.shard_select(sl, w.params, r * width, w.vocab, history_ids=hist, history_offsets=w.history_offsets,
                            uniforms=uni)
        ranks[0].shard_gather_local(ranks)
        out = ranks[0].shard_finish(w.rows, width, w.params, w.vocab, history_ids=hist, history_offsets=w.history_offsets,
                                    uniforms=uni, want_probs=True, want_flags=True, want_topk=50)
        torch.cuda.synchronize()
        got = {k: v.cpu().numpy() for k, v in out.items()}
    finally:
        for bs in ranks:
            bs.close()
        full.close()
    assert np.array_equal(got["tokens"], ref["tokens"])
    assert np.array_equal(got["topk_ids"][4:], ref["topk_ids"][4:])
    assert np.array_equal(got["topk_logits"][4:], ref["topk_logits"][4:])
    assert np.array_equal(got["topk_probs"][4:], ref["topk_probs"][4:])


def test_and_masks_matches_and_constraint_rules():
    """AndTokenConstraint semantics (AndTokenConstraintTests.cs:132-216): intersection of the inners,
    a dead inner is skipped, an empty intersection or no live inner leaves the row unmasked."""
    import torch
    from opentail.stingray_b200 import BatchSampler

    rng = np.random.default_rng(9)
    for vocab in (70, 1000, 151936, 262144):
        words = (vocab + 31) // 32
        rows, K = 7, 3
        m = rng.integers(0, 2 ** 32, (K, rows, words), dtype=np.uint64).astype(np.uint32)
        m[0, 1] = 0                                   # a dead inner in row 1
        m[:, 2] = 0                                   # every inner dead in row 2
        m[0, 3] = 0x55555555; m[1, 3] = 0xAAAAAAAA    # empty intersection in row 3
        m[:, 4] = 0; m[0, 4, words - 1] = 1 << 31     # only a bit beyond the vocabulary (when vocab % 32 != 0)
        m[1, 5] = 0xFFFFFFFF                          # an inner that allows everything
        bs = BatchSampler(max_rows=rows, max_vocab=vocab, max_history=1, max_top_k=8)
        out, uses = bs.and_masks(torch.from_numpy(m.view(np.int32)).cuda(), vocab)
        out = out.cpu().numpy().view(np.uint32)
        uses = uses.cpu().numpy()
        bs.close()
        tail = ((1 << (vocab & 31)) - 1) if vocab & 31 else 0xFFFFFFFF
        for r in range(rows):
            want, masking = orc.and_masks([m[k, r] for k in range(K)], vocab)
            assert bool(uses[r]) == masking, (vocab, r)
            got = out[r].copy()
            got[-1] &= tail
            want[-1] &= tail
            assert np.array_equal(got, want), (vocab, r)
