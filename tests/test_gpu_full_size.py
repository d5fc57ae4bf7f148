"""The benchmark configurations at their stated sizes, every row compared with the CPU oracle:
C2 256 x 151,936 fp32 (mixed parameters, 512-token histories), C3 64 x 262,144 bf16 with masks,
C4 32 sequences x (9 target + 8 draft) x 151,936 with oracle-drawn draft tokens, and a 512-row
shard of C5 (256,000 columns, top-k 50).  A sampled id may differ from the oracle's only where the
oracle itself reports the draw within 1e-6 of a CDF boundary; both counts are printed."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import parity

pytestmark = pytest.mark.gpu


def _run(w, want_topk, max_history, budget):
    from opentail.stingray_b200 import BatchSampler

    bs = BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=max_history, max_top_k=max(want_topk, 1))
    try:
        gpu = parity.run_gpu(bs, w, want_topk=want_topk)
    finally:
        bs.close()
    stats = parity.compare(w, gpu)
    print(f"{w.name}: {stats}")
    assert stats["mismatch"] == stats["boundary_draws"] <= budget, stats
    return stats, gpu


def test_config2_all_256_rows():
    from opentail.stingray_b200 import workloads as W

    stats, _ = _run(W.config2(), 100, 512, 2)
    assert stats["rows"] == 256 and stats["paths"].get(2, 0) > 100 and stats["paths"].get(3, 0) > 30


def test_config3_all_64_rows_bf16_masked():
    from opentail.stingray_b200 import workloads as W

    w = W.config3()
    stats, gpu = _run(w, 0, 1, 2)
    assert stats["rows"] == 64 and stats["paths"] == {3: 64}
    allowed = np.unpackbits(w.mask.view(np.uint8), axis=1, bitorder="little")
    assert all(allowed[r, gpu["tokens"][r]] == 1 for r in range(w.rows)), "a masked token was sampled"


def test_config5_shard_of_512_rows():
    from opentail.stingray_b200 import workloads as W

    stats, _ = _run(W.config5(rows=512), 50, 256, 2)
    assert stats["rows"] == 512 and stats["paths"] == {2: 512}


def test_config4_all_32_sequences():
    import torch
    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import workloads as W

    par = W._params(1)
    op = orc.OrcParams(*[par[0][n].item() for n in par.dtype.names])

    def draw(draft, u):
        toks = np.zeros(u.shape, np.int32)
        for s in range(u.shape[0]):
            for i in range(u.shape[1]):
                toks[s, i] = orc.sample_with_distribution(draft[s, i], op, float(u[s, i]))[0]
        return toks

    w = W.config4(draw_tokens=draw)
    n_seq, lp1, vocab = w.target.shape
    L = lp1 - 1
    assert (n_seq, L, vocab) == (32, 8, W.V_QWEN)
    bs = BatchSampler(max_rows=n_seq * lp1, max_vocab=vocab, max_history=1, max_top_k=8, max_spec_draft=L)
    try:
        out = bs.spec_verify(torch.from_numpy(w.target).cuda(), torch.from_numpy(w.draft).cuda(), w.draft_tokens,
                             w.params, w.uniforms, want_probs=True)
        torch.cuda.synchronize()
        acc, corr = out["accepted"].cpu().numpy(), out["correction"].cpu().numpy()
        ap = out["accept_probs"].cpu().numpy()
    finally:
        bs.close()
    boundary = mismatch = 0
    for s in range(n_seq):
        want_acc, want_corr, want_ap, tr = orc.spec_step_sampled(
            w.target[s], w.draft[s], w.draft_tokens[s], op, w.uniforms[s, :L], w.uniforms[s, L:])
        tested = min(want_acc + 1, L)
        np.testing.assert_allclose(ap[s, :tested], want_ap[:tested], rtol=2e-5, atol=1e-30, err_msg=f"seq {s}")
        if acc[s] != want_acc:
            i = min(acc[s], want_acc)  # an accept test within tolerance of its uniform may flip
            assert abs(float(w.uniforms[s, i]) - float(want_ap[i])) <= 2e-5 * max(float(want_ap[i]), 1e-30), f"seq {s}"
            mismatch += 1
            boundary += 1
        elif corr[s] != want_corr:
            mismatch += 1
            assert tr.margin <= parity.BOUNDARY, f"seq {s}: correction {corr[s]} != {want_corr}, margin {tr.margin}"
            boundary += 1
    print(f"c4_spec_verify: sequences {n_seq} mismatch {mismatch} boundary {boundary} accepted mean {acc.mean():.2f}")
    assert mismatch == boundary <= 2
