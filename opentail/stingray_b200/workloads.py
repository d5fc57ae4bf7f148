"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

No public dataset or model is involved: the reference publishes no sampler benchmark, so every
configuration is generated here (NumPy PCG64, fixed draw order: logits, boosted ids, histories,
per-row parameters, masks, uniforms).  ``rows``/``vocab`` can be reduced for parity tests; the
defaults are the full sizes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from .sampler import PARAMS_DTYPE

V_QWEN = 151_936
V_GEMMA = 262_144
V_LARGE = 256_000


@dataclass
class SampleWorkload:
    name: str
    logits: np.ndarray                 # float32 [rows, vocab] or uint16 (bf16 bits)
    params: np.ndarray                 # PARAMS_DTYPE [rows]
    uniforms: np.ndarray               # float32 [rows]
    history_ids: Optional[np.ndarray] = None
    history_offsets: Optional[np.ndarray] = None
    mask: Optional[np.ndarray] = None  # uint32 [rows, vocab/32]

    @property
    def rows(self):
        return self.logits.shape[0]

    @property
    def vocab(self):
        return self.logits.shape[1]

    def algorithmic_bytes(self) -> int:
        """Bytes one step must touch: every input once, every output once."""
        b = self.logits.nbytes + self.params.nbytes + self.uniforms.nbytes + 4 * self.rows
        if self.history_ids is not None:
            b += self.history_ids.nbytes
        if self.mask is not None:
            b += self.mask.nbytes
        return b


def uniforms24(rng, n) -> np.ndarray:
    """float32 uniforms (j + 0.5) / 2^24: never 0 or 1, exactly representable."""
    j = rng.integers(0, 1 << 24, size=n)
    return ((j.astype(np.float64) + 0.5) / float(1 << 24)).astype(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def _params(rows, **kw) -> np.ndarray:
    p = np.zeros(rows, PARAMS_DTYPE)
    p["temperature"], p["top_p"], p["repetition_penalty"], p["repeat_last_n"] = 1.0, 1.0, 1.0, 64
    for k, v in kw.items():
        p[k] = v
    return p


def _csr(hist: np.ndarray):
    rows, h = hist.shape
    return hist.reshape(-1).astype(np.int32), (np.arange(rows + 1) * h).astype(np.int32)


def zipf_ids(rng, rows, count, vocab, s=1.1) -> np.ndarray:
    """Truncated Zipf(s) over ranks 1..vocab by inverse CDF; id = rank - 1."""
    w = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    u = rng.random((rows, count))
    return np.minimum(np.searchsorted(cdf, u), vocab - 1).astype(np.int32)


def config1(vocab=V_QWEN, seed=0, greedy=False) -> SampleWorkload:
    """Single row, CPU-runnable: N(0, 3^2) with 16 seeded ids boosted by +8, 64-token history,
    T 0.8, repetition 1.1, top-k 40, top-p 0.95, min-p 0.05."""
    rng = np.random.default_rng(seed)
    logits = rng.normal(0.0, 3.0, (1, vocab)).astype(np.float32)
    boosted = rng.choice(vocab, 16, replace=False)
    logits[0, boosted] += np.float32(8.0)
    hist = rng.integers(0, vocab, (1, 64)).astype(np.int32)
    p = _params(1, temperature=0.0 if greedy else 0.8, repetition_penalty=1.1, repeat_last_n=64,
                top_k=40, top_p=0.95, min_p=0.05)
    ids, off = _csr(hist)
    return SampleWorkload("c1_single_row", logits, p, uniforms24(rng, 1), ids, off)


def config2(rows=256, vocab=V_QWEN, seed=1, history=512) -> SampleWorkload:
    """Batched server decode: N(0, 2.5^2); per row T~U[0.3,1.2], top-k in {0,20,50,100},
    top-p~U[0.8,1.0], frequency 0.5, presence 0.3 over a Zipf(1.1) history of 512 ids."""
    rng = np.random.default_rng(seed)
    logits = rng.normal(0.0, 2.5, (rows, vocab)).astype(np.float32)
    hist = zipf_ids(rng, rows, history, vocab)
    p = _params(rows, frequency_penalty=0.5, presence_penalty=0.3)
    p["temperature"] = rng.uniform(0.3, 1.2, rows).astype(np.float32)
    p["top_k"] = rng.choice(np.array([0, 20, 50, 100]), rows)
    p["top_p"] = rng.uniform(0.8, 1.0, rows).astype(np.float32)
    ids, off = _csr(hist)
    return SampleWorkload("c2_server_decode", logits, p, uniforms24(rng, rows), ids, off)


def config3(rows=64, vocab=V_GEMMA, seed=2) -> SampleWorkload:
    """Grammar-constrained: bf16 N(0, 3^2); per-row allowed-token bitmask of density log-uniform in
    [0.1 %, 30 %] with at least one bit set; T 0.7, top-p 0.9."""
    rng = np.random.default_rng(seed)
    logits = to_bf16_bits(rng.normal(0.0, 3.0, (rows, vocab)).astype(np.float32))
    words = (vocab + 31) // 32
    mask = np.zeros((rows, words), np.uint32)
    dens = np.exp(rng.uniform(np.log(0.001), np.log(0.30), rows))
    for r in range(rows):
        n = max(1, int(round(dens[r] * vocab)))
        ids = rng.choice(vocab, n, replace=False)
        np.bitwise_or.at(mask[r], ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
    p = _params(rows, temperature=0.7, top_p=0.9)
    return SampleWorkload("c3_grammar_masked", logits, p, uniforms24(rng, rows), mask=mask)


@dataclass
class SpecWorkload:
    name: str
    target: np.ndarray        # float32 [n_seq, L + 1, vocab]
    draft: np.ndarray         # float32 [n_seq, L, vocab]
    draft_tokens: np.ndarray  # int32 [n_seq, L]
    params: np.ndarray        # PARAMS_DTYPE [n_seq]
    uniforms: np.ndarray      # float64 [n_seq, L + 2]

    def algorithmic_bytes(self) -> int:
        return (self.target.nbytes + self.draft.nbytes + self.draft_tokens.nbytes +
                self.uniforms.nbytes + 8 * self.target.shape[0])


def config4(n_seq=32, n_draft=8, vocab=V_QWEN, seed=3, draw_tokens=None) -> SpecWorkload:
    """Speculative verification: draft logits N(0, 3^2), target = draft + N(0, 0.5^2) (plus one
    bonus row), temperature 1.  Draft tokens are drawn from softmax(draft row) with seeded
    uniforms by ``draw_tokens(draft_rows, uniforms) -> ids`` (the oracle's inverse-CDF rule); when
    it is None a plain NumPy inverse CDF in float64 is used."""
    rng = np.random.default_rng(seed)
    draft = rng.normal(0.0, 3.0, (n_seq, n_draft, vocab)).astype(np.float32)
    target = np.empty((n_seq, n_draft + 1, vocab), np.float32)
    target[:, :n_draft] = draft + rng.normal(0.0, 0.5, (n_seq, n_draft, vocab)).astype(np.float32)
    target[:, n_draft] = rng.normal(0.0, 3.0, (n_seq, vocab)).astype(np.float32)
    u_draw = uniforms24(rng, n_seq * n_draft).reshape(n_seq, n_draft)
    if draw_tokens is None:
        toks = np.empty((n_seq, n_draft), np.int32)
        for s in range(n_seq):
            for i in range(n_draft):
                z = draft[s, i].astype(np.float64)
                e = np.exp(z - z.max())
                cdf = np.cumsum(e / e.sum())
                toks[s, i] = min(int(np.searchsorted(cdf, float(u_draw[s, i]))), vocab - 1)
    else:
        toks = draw_tokens(draft, u_draw).astype(np.int32)
    uni = uniforms24(rng, n_seq * (n_draft + 2)).reshape(n_seq, n_draft + 2).astype(np.float64)
    return SpecWorkload("c4_spec_verify", target, draft, toks, _params(n_seq), uni)


def config5(rows=4096, vocab=V_LARGE, seed=4, history=256) -> SampleWorkload:
    """Large multi-GPU sampling: N(0, 3^2), top-k 50, top-p 0.9, T 1.0, repetition 1.05 over
    256-token uniform histories (whole history in the window)."""
    rng = np.random.default_rng(seed)
    logits = rng.standard_normal((rows, vocab), dtype=np.float32) * np.float32(3.0)
    hist = rng.integers(0, vocab, (rows, history)).astype(np.int32)
    p = _params(rows, top_k=50, top_p=0.9, repetition_penalty=1.05, repeat_last_n=0)
    ids, off = _csr(hist)
    return SampleWorkload("c5_large_batch", logits, p, uniforms24(rng, rows), ids, off)
