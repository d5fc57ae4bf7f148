"""Shared helpers of the parity tests: run a workload through the CUDA library and through the CPU
oracle on the same inputs, and compare by the rules of the sampling contract:

* greedy argmax, top-k candidate ids and their penalised logits: bit-exact;
* probabilities: within 1e-5 relative;
* sampled ids: identical for the same uniform, except draws within 1e-6 of a CDF boundary,
  which are counted and returned.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle as orc

REL_TOL = 1e-5
BOUNDARY = 1e-6


def to_device(w):
    import torch

    dev = {}
    lg = torch.from_numpy(w.logits.view(np.int16) if w.logits.dtype == np.uint16 else w.logits).cuda()
    dev["logits"] = lg.view(torch.bfloat16) if w.logits.dtype == np.uint16 else lg
    dev["uniforms"] = torch.from_numpy(w.uniforms).cuda()
    if w.history_ids is not None:
        dev["history_ids"] = torch.from_numpy(w.history_ids).cuda()
    if w.mask is not None:
        dev["mask"] = torch.from_numpy(w.mask.view(np.int32)).cuda()
    return dev


def run_gpu(bs, w, dev=None, want_topk=0):
    dev = dev or to_device(w)
    kw = dict(uniforms=dev["uniforms"], want_probs=True, want_flags=True, want_topk=want_topk)
    if w.history_ids is not None:
        kw.update(history_ids=dev["history_ids"], history_offsets=w.history_offsets)
    if w.mask is not None:
        kw.update(mask=dev["mask"])
    out = bs.sample_rows(dev["logits"], w.params, **kw)
    import torch

    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in out.items()}


def oracle_rows(w, sum_mode=0):
    return orc.sample_rows(w.logits, w.params, w.uniforms.astype(np.float64), w.history_ids,
                           w.history_offsets, w.mask, sum_mode=sum_mode)


def row_logits_f32(w, r):
    row = w.logits[r]
    if row.dtype == np.uint16:
        row = (row.astype(np.uint32) << 16).view(np.float32)
    if w.mask is not None:
        row = orc.apply_mask(row, w.mask[r])
    return row


def row_history(w, r):
    if w.history_ids is None:
        return None
    return w.history_ids[w.history_offsets[r]:w.history_offsets[r + 1]]


def compare(w, gpu, check_topk=True):
    """Returns a dict of counters; raises AssertionError on a contract violation."""
    tokens, traces = oracle_rows(w)
    flags = gpu["flags"].view(np.uint32)
    stats = {"rows": w.rows, "boundary_draws": 0, "tie_rows": 0, "mismatch": 0, "paths": {}}
    for r in range(w.rows):
        path = int(traces["path"][r])
        stats["paths"][path] = stats["paths"].get(path, 0) + 1
        assert int(flags[r] & 7) == path, f"row {r}: path {flags[r] & 7} != oracle {path}"
        if path in (0, 1, 4):
            assert gpu["tokens"][r] == tokens[r], f"row {r}: greedy token {gpu['tokens'][r]} != {tokens[r]}"
            continue
        p = orc.OrcParams(*[w.params[r][n].item() for n in w.params.dtype.names])
        if path == 2 and check_topk:
            k = int(w.params["top_k"][r])
            res = orc.sample(row_logits_f32(w, r), p, float(w.uniforms[r]), history=row_history(w, r))
            np.testing.assert_array_equal(gpu["topk_ids"][r, :k], res.cand_ids[:k], err_msg=f"row {r} top-k ids")
            assert np.array_equal(gpu["topk_logits"][r, :k], res.cand_vals[:k]), f"row {r} penalised logits"
            np.testing.assert_allclose(gpu["topk_probs"][r, :k], res.cand_probs[:k], rtol=REL_TOL, atol=1e-30,
                                       err_msg=f"row {r} top-k probs")
        if flags[r] & (1 << 4) or traces["tie_at_cutoff"][r]:
            stats["tie_rows"] += 1
        if gpu["tokens"][r] != tokens[r]:
            stats["mismatch"] += 1
            m = float(traces["margin"][r])
            assert m <= BOUNDARY, (f"row {r}: token {gpu['tokens'][r]} != oracle {tokens[r]} with the draw "
                                   f"{m:.3e} away from a CDF boundary (path {path})")
            stats["boundary_draws"] += 1
        else:
            np.testing.assert_allclose(gpu["probs"][r], traces["prob"][r], rtol=2e-5, atol=1e-30,
                                       err_msg=f"row {r} token prob")
    return stats
