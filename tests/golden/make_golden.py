"""Generates tests/golden/sampler_golden.json: outputs of the CPU oracle on seeded inputs.

The reference's own tests carry no golden vectors for large vocabularies (their inline literals are
restated in tests/test_oracle_kat.py), and the reference cannot be run here, so these vectors pin the
oracle's behaviour over time rather than the reference's: a later change to the oracle or to the
workload generators that alters any token shows up as a diff of this file.  Inputs are not stored;
they are regenerated from the seeds below and guarded by a SHA-256 of their bytes.

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from opentail.stingray_b200 import workloads as W  # noqa: E402
from oracle import oracle as orc  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sampler_golden.json")


def sample_cases():
    """name -> workload; sizes the oracle finishes in seconds."""
    return {
        "c1_single_row": W.config1(),
        "c1_greedy": W.config1(greedy=True),
        "c2_server_decode_24rows": W.config2(rows=24),
        "c3_grammar_masked_6rows": W.config3(rows=6),
        "c5_large_batch_8rows": W.config5(rows=8),
    }


def spec_case():
    p = orc.make_params()

    def draw(draft, u):
        out = np.empty(u.shape, np.int32)
        for s in range(u.shape[0]):
            for i in range(u.shape[1]):
                out[s, i] = orc.sample_with_distribution(draft[s, i], p, float(u[s, i]))[0]
        return out

    return W.config4(n_seq=4, n_draft=4, vocab=32000, draw_tokens=draw)


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def golden_for(w) -> dict:
    tokens, tr = orc.sample_rows(w.logits, w.params, w.uniforms.astype(np.float64), w.history_ids,
                                 w.history_offsets, w.mask)
    return {
        "rows": int(w.rows), "vocab": int(w.vocab),
        "inputs_sha256": digest(w.logits, w.params, w.uniforms, w.history_ids, w.history_offsets, w.mask),
        "tokens": [int(t) for t in tokens],
        "paths": [int(x) for x in tr["path"]],
        "token_prob_f32_bits": [int(np.float32(x).view(np.uint32)) for x in tr["prob"]],
    }


def golden_spec(w) -> dict:
    p = orc.make_params()
    L = w.draft_tokens.shape[1]
    acc, corr = [], []
    for s in range(w.target.shape[0]):
        a, c, _, _ = orc.spec_step_sampled(w.target[s], w.draft[s], w.draft_tokens[s], p,
                                           w.uniforms[s, :L], w.uniforms[s, L:])
        acc.append(int(a))
        corr.append(int(c))
    return {"n_seq": int(w.target.shape[0]), "n_draft": int(L), "vocab": int(w.target.shape[2]),
            "inputs_sha256": digest(w.target, w.draft, w.draft_tokens, w.uniforms),
            "draft_tokens": w.draft_tokens.tolist(), "accepted": acc, "correction": corr}


def main():
    doc = {"sample": {k: golden_for(w) for k, w in sample_cases().items()},
           "spec": {"c4_spec_verify_4seq": golden_spec(spec_case())}}
    with open(OUT, "w") as f:
        json.dump(doc, f, indent=1, sort_keys=True)
        f.write("\n")
    print(f"wrote {OUT}")


if __name__ == "__main__":
    main()
