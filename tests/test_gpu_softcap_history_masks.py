"""GPU tests of the steps either side of the sampler that were moved into it:

* the final-logit soft cap applied on load (llm_softcap_inplace, CudaTextKernels.cs:374-383): identical,
  bit for bit, to sampling soft-capped logits that the same CUDA math produced beforehand, and within the
  sampling contract of the CPU oracle run on tanhf-capped logits;
* device-resident histories (the engine's per-sequence PreviousTokens, ContinuousBatchingEngine.cs:650,
  :1280): a decode loop that appends its own output on the device equals the oracle fed host lists;
* the bitmask cache and its AND / OR composition (AndTokenConstraint.cs:44-86) against numpy.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import parity

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bs():
    from opentail.stingray_b200 import BatchSampler

    s = BatchSampler(max_rows=64, max_vocab=151936, max_history=512, max_top_k=512, max_spec_draft=4,
                     max_cached_masks=6)
    yield s
    s.close()


def _capped_on_gpu(x, cap):
    """tanh(x / cap) * cap with CUDA's own tanhf and a true division, as the reference kernel computes it."""
    import torch

    xf = x.float()
    return torch.tanh(xf / torch.full_like(xf, cap)) * cap


@pytest.mark.parametrize("bf16", [False, True])
def test_softcap_on_load_equals_sampling_capped_logits(bs, bf16):
    import torch
    from opentail.stingray_b200 import workloads as W

    w = W.config2(rows=48, seed=21)
    dev = parity.to_device(w)
    x = dev["logits"] * 6.0  # spread the logits so that the cap (30) bends them visibly
    if bf16:
        x = x.to(torch.bfloat16)
    cap = 30.0
    kw = dict(uniforms=dev["uniforms"], want_probs=True, want_flags=True, want_topk=int(w.params["top_k"].max()),
              history_ids=dev["history_ids"], history_offsets=w.history_offsets)
    fused = bs.sample_rows(x, w.params, softcap=cap, **kw)
    plain = bs.sample_rows(_capped_on_gpu(x, cap), w.params, **kw)
    for name in ("tokens", "probs", "flags"):
        assert torch.equal(fused[name], plain[name]), name
    on_topk_path = (fused["flags"].cpu().numpy().view(np.uint32) & 7) == 2  # the other rows' slots are not written
    assert on_topk_path.any()
    for name in ("topk_ids", "topk_logits", "topk_probs"):
        for r in np.nonzero(on_topk_path)[0]:
            k = int(w.params["top_k"][r])
            assert torch.equal(fused[name][r, :k], plain[name][r, :k]), (name, r)
    d_fused = bs.build_distribution(x[:8], w.params[:8], softcap=cap)
    d_plain = bs.build_distribution(_capped_on_gpu(x[:8], cap), w.params[:8])
    assert torch.equal(d_fused, d_plain)
    # and the cap is really applied: the uncapped distributions differ
    assert not torch.equal(d_fused, bs.build_distribution(x[:8].float(), w.params[:8]))


def test_softcap_against_the_oracle(bs):
    import torch
    from opentail.stingray_b200 import workloads as W

    w = W.config2(rows=32, seed=22)
    cap = 30.0
    raw = (w.logits * np.float32(6.0)).astype(np.float32)
    dev = parity.to_device(w)
    out = bs.sample_rows(torch.from_numpy(raw).cuda(), w.params, uniforms=dev["uniforms"], want_probs=True, want_flags=True,
                         history_ids=dev["history_ids"], history_offsets=w.history_offsets, softcap=cap)
    tokens = out["tokens"].cpu().numpy()
    probs = out["probs"].cpu().numpy()
    flags = out["flags"].cpu().numpy().view(np.uint32)
    capped = orc.softcap(raw, cap)
    want, traces = orc.sample_rows(capped, w.params, w.uniforms.astype(np.float64), w.history_ids, w.history_offsets, None)
    near = 0
    for r in range(w.rows):
        assert int(flags[r] & 7) == int(traces["path"][r])
        if tokens[r] != want[r]:
            # tanhf of the host's libm and of CUDA may differ in the last bit: allowed only where the oracle
            # itself says that the draw, the arg-max or the cut sat on a boundary
            assert traces["path"][r] not in (0, 1, 4), f"row {r}: greedy token differs"
            assert float(traces["margin"][r]) <= 1e-5, f"row {r}: token {tokens[r]} != {want[r]}"
            near += 1
        else:
            np.testing.assert_allclose(probs[r], traces["prob"][r], rtol=1e-4, atol=1e-30, err_msg=f"row {r}")
    assert near <= 2
    dist = bs.build_distribution(torch.from_numpy(raw[:6]).cuda(), w.params[:6], softcap=cap).cpu().numpy()
    for r in range(6):
        if w.params["temperature"][r] <= 0:
            continue
        p = orc.OrcParams(*[w.params[r][n].item() for n in w.params.dtype.names])
        ref, tr = orc.build_filtered_distribution(capped[r], p)
        both = (dist[r] > 0) & (ref > 0)
        assert both.sum() >= (ref > 0).sum() - 1  # a last-bit difference may move a cut by one token
        np.testing.assert_allclose(dist[r][both], ref[both], rtol=1e-4)


def test_spec_verify_softcaps(bs):
    import torch
    from opentail.stingray_b200 import workloads as W

    w = W.config4(n_seq=6, n_draft=4, vocab=32000, seed=5)
    t = torch.from_numpy(w.target).cuda() * 5.0
    d = torch.from_numpy(w.draft).cuda() * 5.0
    dt = torch.from_numpy(w.draft_tokens).cuda()
    u = torch.from_numpy(w.uniforms).cuda()
    fused = bs.spec_verify(t, d, dt, w.params, u, want_probs=True, target_softcap=30.0, draft_softcap=20.0)
    plain = bs.spec_verify(_capped_on_gpu(t, 30.0), _capped_on_gpu(d, 20.0), dt, w.params, u, want_probs=True)
    for name in ("accepted", "correction", "accept_probs", "flags"):
        assert torch.equal(fused[name], plain[name]), name


def _decode_loop(bs, rng, rows, vocab, params, steps, cap_hist, seed_hist):
    """`steps` sampling steps on fresh logits each; returns the tokens of every step."""
    import torch

    bs.history_reset()
    for r, h in enumerate(seed_hist):
        bs.history_load(r, h)
    got, all_logits, all_u = [], [], []
    for s in range(steps):
        logits = rng.normal(0, 2.0, (rows, vocab)).astype(np.float32)
        u = rng.random(rows).astype(np.float32)
        out = bs.sample_rows(torch.from_numpy(logits).cuda(), params, uniforms=torch.from_numpy(u).cuda(), history_ring=True,
                             want_flags=True)
        bs.history_append(out["tokens"])
        got.append((out["tokens"].cpu().numpy(), out["flags"].cpu().numpy().view(np.uint32)))
        all_logits.append(logits)
        all_u.append(u)
    return got, all_logits, all_u


def test_device_histories_follow_a_decode_loop():
    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import workloads as W

    rng = np.random.default_rng(9)
    rows, vocab, steps, cap_hist = 12, 8192, 10, 16
    p = W._params(rows)
    p["temperature"] = [0.0, 0.8, 0.9, 1.0, 0.7, 0.0, 1.1, 0.8, 0.9, 1.0, 0.6, 0.8]
    p["top_k"] = [0, 40, 0, 20, 50, 0, 0, 5, 40, 0, 64, 0]
    p["top_p"] = [1.0, 0.9, 0.9, 1.0, 0.95, 1.0, 0.8, 1.0, 0.9, 1.0, 0.9, 0.95]
    p["repetition_penalty"] = [1.3, 1.2, 1.1, 1.5, 1.0, 1.2, 1.3, 1.1, 1.2, 1.0, 1.4, 1.2]
    p["repeat_last_n"] = 8  # inside what a 16-entry history keeps after it starts dropping
    seed_hist = [rng.integers(0, vocab, int(n)).astype(np.int32) for n in rng.integers(0, cap_hist - 2, rows)]
    bs = BatchSampler(max_rows=rows, max_vocab=vocab, max_history=cap_hist, max_top_k=64)
    try:
        got, logits, us = _decode_loop(bs, rng, rows, vocab, p, steps, cap_hist, seed_hist)
        lists = [list(h) for h in seed_hist]
        dropped = False
        for s in range(steps):
            tokens, flags = got[s]
            for r in range(rows):
                op = orc.OrcParams(*[p[r][n].item() for n in p.dtype.names])
                res = orc.sample(logits[s][r], op, float(us[s][r]), history=np.array(lists[r], np.int32))
                if tokens[r] != res.token:
                    assert res.trace.margin <= parity.BOUNDARY, f"step {s} row {r}: {tokens[r]} != {res.token}"
                # the device appended what the device sampled
                lists[r].append(int(tokens[r]))
                dropped |= len(lists[r]) > cap_hist
        assert [bs.history_length(r) for r in range(rows)] == [min(len(h), cap_hist) for h in lists]
        assert dropped, "the loop was meant to run the histories past their capacity"
        # a row whose penalties count the whole history cannot be served once tokens were dropped
        p2 = p.copy()
        p2["presence_penalty"] = 0.5
        import torch
        from opentail.stingray_b200 import StingrayError

        with pytest.raises(StingrayError) as e:
            bs.sample_rows(torch.from_numpy(logits[0]).cuda(), p2, uniforms=torch.from_numpy(us[0]).cuda(), history_ring=True)
        assert e.value.code == 3
    finally:
        bs.close()


def test_device_histories_inactive_rows_and_full_window(bs):
    import torch
    from opentail.stingray_b200 import workloads as W

    rng = np.random.default_rng(10)
    rows, vocab = 8, 151936
    p = W._params(rows)
    p["temperature"] = 0.9
    p["top_k"] = [50, 0, 50, 0, 50, 0, 50, 0]
    p["top_p"] = 0.9
    p["repetition_penalty"] = 1.2
    p["presence_penalty"] = 0.3
    p["frequency_penalty"] = 0.2
    p["repeat_last_n"] = 0  # whole history
    bs.history_reset()
    lists = [[] for _ in range(rows)]
    for s in range(5):
        logits = rng.normal(0, 2.0, (rows, vocab)).astype(np.float32)
        u = rng.random(rows).astype(np.float32)
        active = (rng.random(rows) < 0.7).astype(np.uint8)
        out = bs.sample_rows(torch.from_numpy(logits).cuda(), p, uniforms=torch.from_numpy(u).cuda(), history_ring=True)
        bs.history_append(out["tokens"], active=active)
        tokens = out["tokens"].cpu().numpy()
        for r in range(rows):
            op = orc.OrcParams(*[p[r][n].item() for n in p.dtype.names])
            res = orc.sample(logits[r], op, float(u[r]), history=np.array(lists[r], np.int32))
            if tokens[r] != res.token:
                assert res.trace.margin <= parity.BOUNDARY, f"step {s} row {r}"
            if active[r]:
                lists[r].append(int(tokens[r]))
        assert [bs.history_length(r) for r in range(rows)] == [len(h) for h in lists]


def _np_compose(masks, vocab, op):
    """numpy statement of the composition: masks is a list of word arrays (or None for an empty slot)."""
    words = (vocab + 31) // 32
    tail = np.uint32((1 << (vocab & 31)) - 1) if vocab & 31 else np.uint32(0xFFFFFFFF)

    def trimmed(m):
        t = m[:words].copy()
        t[-1] &= tail
        return t

    alive = [m for m in masks if m is not None and trimmed(m).any()]
    ones = np.full(words, 0xFFFFFFFF, np.uint32)
    if not alive:
        return ones, 0
    acc = alive[0][:words].copy()
    for m in alive[1:]:
        acc = (acc & m[:words]) if op == "and" else (acc | m[:words])
    if not trimmed(acc).any():
        return ones, 0
    return acc, 1


def test_mask_cache_compose(bs):
    from opentail.stingray_b200 import StingrayError

    rng = np.random.default_rng(3)
    vocab = 151936 - 5  # a ragged last word
    words = (vocab + 31) // 32
    store = {}
    for key in (11, 12, 13, 14):
        m = rng.integers(0, 1 << 32, words, dtype=np.uint64).astype(np.uint32)
        if key == 13:
            m &= rng.integers(0, 1 << 32, words, dtype=np.uint64).astype(np.uint32)  # sparser
        store[key] = m
    store[15] = np.zeros(words, np.uint32)                      # a dead inner: allows nothing
    store[16] = np.zeros(words, np.uint32); store[16][7] = 1 << 3   # allows one token
    for k, m in store.items():
        bs.mask_cache_put(k, m, vocab)
    assert all(bs.mask_cache_contains(k) for k in store) and not bs.mask_cache_contains(99)
    keys = np.array([[11, 12, 0], [11, 15, 13], [0, 0, 0], [15, 0, 0], [16, 11, 12], [14, 0, 0], [16, 13, 12]], np.uint64)
    for op in ("and", "or"):
        out, uses = bs.mask_compose(keys, vocab, op)
        out = out.cpu().numpy().view(np.uint32)
        uses = uses.cpu().numpy()
        for r in range(keys.shape[0]):
            want, want_uses = _np_compose([store[int(k)] if k else None for k in keys[r]], vocab, op)
            assert uses[r] == want_uses, (op, r)
            if want_uses:
                # bits beyond the vocabulary in the last word are not part of the contract
                tail = np.uint32((1 << (vocab & 31)) - 1)
                assert np.array_equal(out[r, :-1], want[:-1]) and (out[r, -1] & tail) == (want[-1] & tail), (op, r)
            else:
                assert (out[r] == 0xFFFFFFFF).all(), (op, r)
    # a key that was never stored is an error, and the seventh entry evicts the one used longest ago
    with pytest.raises(StingrayError):
        bs.mask_compose(np.array([[11, 99]], np.uint64), vocab, "and")
    bs.mask_compose(np.array([[11, 12, 13, 15, 16]], np.uint64), vocab, "or")  # 14 is now the stalest
    walked = []
    ran = bs.mask_cache_get_or_put(17, vocab, lambda: walked.append(1) or np.arange(0, vocab, 3))
    assert ran and walked == [1]
    assert not bs.mask_cache_get_or_put(17, vocab, lambda: walked.append(1) or np.arange(0, vocab, 3)) and walked == [1]
    assert not bs.mask_cache_contains(14) and bs.mask_cache_contains(11) and bs.mask_cache_contains(17)
    out, uses = bs.mask_compose(np.array([[17]], np.uint64), vocab, "and")
    got = out.cpu().numpy().view(np.uint32)[0]
    ids = np.arange(0, vocab, 3)
    bits = (got[ids >> 5] >> (ids & 31).astype(np.uint32)) & 1
    assert bits.all() and int(np.unpackbits(got.view(np.uint8)).sum()) == ids.size


def test_composed_mask_feeds_the_sampler(bs):
    """The composed rows go into stg_sample_rows as they are: the sampled token is always allowed."""
    import torch

    rng = np.random.default_rng(4)
    vocab, rows = 151936, 6
    words = (vocab + 31) // 32
    a = np.zeros(words, np.uint32); a[100:400] = 0xFFFFFFFF
    b = np.zeros(words, np.uint32); b[300:700] = 0x0F0F0F0F
    bs.mask_cache_put(21, a, vocab)
    bs.mask_cache_put(22, b, vocab)
    keys = np.array([[21, 22]] * rows, np.uint64)
    mask, uses = bs.mask_compose(keys, vocab, "and")
    from opentail.stingray_b200 import workloads as W

    p = W._params(rows)
    p["temperature"] = [0.0, 0.8, 0.9, 1.0, 0.7, 1.2]
    p["top_k"] = [0, 40, 0, 20, 0, 50]
    p["top_p"] = [1.0, 0.9, 0.9, 1.0, 1.0, 0.95]
    logits = rng.normal(0, 2.0, (rows, vocab)).astype(np.float32)
    u = rng.random(rows).astype(np.float32)
    out = bs.sample_rows(torch.from_numpy(logits).cuda(), p, uniforms=torch.from_numpy(u).cuda(), mask=mask,
                         row_uses_mask=uses.cpu().numpy())
    tokens = out["tokens"].cpu().numpy()
    both = a & b
    want, _ = orc.sample_rows(logits, p, u.astype(np.float64), None, None, np.tile(both, (rows, 1)))
    for r in range(rows):
        assert (both[tokens[r] >> 5] >> (tokens[r] & 31)) & 1
        assert tokens[r] == want[r]
