"""ctypes binding of the CPU oracle (``oracle/sampler_oracle.c``).

TEST INFRASTRUCTURE ONLY: the product package never imports this module.  It is loaded by the
test-suite, by the smoke check and by the benchmark's CPU-baseline leg, as the checker.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libsampler_oracle.so")


class OrcParams(C.Structure):
    """Mirror of ``OrcParams`` (SamplingParams, Engine/Sampler.cs:648-686)."""

    _fields_ = [
        ("temperature", C.c_float),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("repetition_penalty", C.c_float),
        ("presence_penalty", C.c_float),
        ("frequency_penalty", C.c_float),
        ("top_k", C.c_int32),
        ("repeat_last_n", C.c_int32),
    ]


class OrcTrace(C.Structure):
    _fields_ = [
        ("path", C.c_int32),
        ("n_cand", C.c_int32),
        ("kept", C.c_int32),
        ("tie_at_cutoff", C.c_int32),
        ("margin", C.c_float),
        ("prob", C.c_float),
        ("kept_sum", C.c_float),
        ("fallback", C.c_int32),
        ("cut_margin", C.c_float),
    ]


PARAMS_DTYPE = np.dtype(
    [
        ("temperature", "<f4"),
        ("top_p", "<f4"),
        ("min_p", "<f4"),
        ("repetition_penalty", "<f4"),
        ("presence_penalty", "<f4"),
        ("frequency_penalty", "<f4"),
        ("top_k", "<i4"),
        ("repeat_last_n", "<i4"),
    ]
)

TRACE_DTYPE = np.dtype(
    [
        ("path", "<i4"),
        ("n_cand", "<i4"),
        ("kept", "<i4"),
        ("tie_at_cutoff", "<i4"),
        ("margin", "<f4"),
        ("prob", "<f4"),
        ("kept_sum", "<f4"),
        ("fallback", "<i4"),
        ("cut_margin", "<f4"),
    ]
)


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (``make -C oracle``) and return the library path."""
    src = os.path.join(_HERE, "sampler_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _f32p = C.POINTER(C.c_float)
        _i32p = C.POINTER(C.c_int32)
        _lib.orc_softcap_inplace.restype = None
        _lib.orc_softcap_inplace.argtypes = [_f32p, C.c_int64, C.c_float]
        _lib.orc_greedy.restype = C.c_int32
        _lib.orc_greedy.argtypes = [_f32p, C.c_int32]
        _lib.orc_sample.restype = C.c_int32
        _lib.orc_sample.argtypes = [
            _f32p, C.c_int32, C.POINTER(OrcParams), _i32p, C.c_int32, _i32p, _f32p, C.c_int32,
            C.c_int, C.c_double, C.POINTER(OrcTrace), _i32p, _f32p, _f32p, _f32p,
        ]
        _lib.orc_build_filtered_distribution.restype = None
        _lib.orc_build_filtered_distribution.argtypes = [
            _f32p, C.c_int32, C.POINTER(OrcParams), _i32p, C.c_int32, _i32p, _f32p, C.c_int32,
            C.c_int, _f32p, _i32p,
        ]
        _lib.orc_build_filtered_distribution_ex.restype = None
        _lib.orc_build_filtered_distribution_ex.argtypes = [
            _f32p, C.c_int32, C.POINTER(OrcParams), _i32p, C.c_int32, _i32p, _f32p, C.c_int32,
            C.c_int, _f32p, _i32p, _f32p,
        ]
        _lib.orc_sample_with_distribution.restype = C.c_int32
        _lib.orc_sample_with_distribution.argtypes = [
            _f32p, C.c_int32, C.POINTER(OrcParams), _i32p, C.c_int32, C.c_int, C.c_double, _f32p,
            C.POINTER(OrcTrace),
        ]
        _lib.orc_sample_from_probs.restype = C.c_int32
        _lib.orc_sample_from_probs.argtypes = [_f32p, C.c_int32, C.c_double, C.POINTER(OrcTrace)]
        _lib.orc_resample_residual.restype = C.c_int32
        _lib.orc_resample_residual.argtypes = [
            _f32p, _f32p, C.c_int32, C.POINTER(C.c_double), _i32p, C.POINTER(OrcTrace)]
        _lib.orc_spec_step_sampled.restype = C.c_int32
        _lib.orc_spec_step_sampled.argtypes = [
            _f32p, _f32p, C.c_int32, C.c_int32, _i32p, C.POINTER(OrcParams), C.c_int,
            C.POINTER(C.c_double), C.POINTER(C.c_double), C.c_int32, C.c_float, _i32p, _f32p,
            C.POINTER(OrcTrace),
        ]
        _lib.orc_spec_greedy_accept.restype = C.c_int32
        _lib.orc_spec_greedy_accept.argtypes = [_f32p, C.c_int32, C.c_int32, _i32p]
        _lib.orc_softmax_prob_at.restype = C.c_float
        _lib.orc_softmax_prob_at.argtypes = [_f32p, C.c_int32, C.c_int32]
        _lib.orc_mtp_accept.restype = C.c_int32
        _lib.orc_mtp_accept.argtypes = [_f32p, C.c_int32, C.c_int32, C.c_float, _f32p]
        _lib.orc_apply_mask.restype = None
        _lib.orc_apply_mask.argtypes = [_f32p, C.c_int32, C.POINTER(C.c_uint32)]
        _lib.orc_and_masks.restype = C.c_int32
        _lib.orc_and_masks.argtypes = [C.POINTER(C.POINTER(C.c_uint32)), C.c_int32, C.c_int32,
                                       C.POINTER(C.c_uint32)]
        _lib.orc_apply_history_penalties.restype = None
        _lib.orc_apply_history_penalties.argtypes = [_f32p, C.c_int32, C.POINTER(OrcParams), _i32p,
                                                     C.c_int32]
        _lib.orc_sample_rows.restype = None
        _lib.orc_sample_rows.argtypes = [
            C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_void_p, _i32p, _i32p,
            C.POINTER(C.c_uint32), C.c_int64, C.POINTER(C.c_double), C.c_int, _i32p, C.c_void_p,
        ]
    return _lib


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _i32(a):
    if a is None:
        return None, None
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(C.POINTER(C.c_int32))


def make_params(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
                repeat_last_n=64, presence_penalty=0.0, frequency_penalty=0.0) -> OrcParams:
    return OrcParams(temperature, top_p, min_p, repetition_penalty, presence_penalty,
                     frequency_penalty, top_k, repeat_last_n)


@dataclass
class SampleResult:
    token: int
    trace: OrcTrace
    cand_ids: np.ndarray | None = None
    cand_vals: np.ndarray | None = None
    cand_probs: np.ndarray | None = None
    probs: np.ndarray | None = None


def softcap(logits, cap: float) -> np.ndarray:
    """A soft-capped copy of ``logits`` (any shape): tanh(x / cap) * cap in float32."""
    a = np.array(logits, dtype=np.float32, order="C", copy=True)
    lib().orc_softcap_inplace(a.ctypes.data_as(C.POINTER(C.c_float)), a.size, cap)
    return a


def greedy(logits) -> int:
    a, p = _f32(logits)
    return lib().orc_greedy(p, a.size)


def sample(logits, params: OrcParams, u: float = 0.5, history=None, bias=None, sum_mode=0,
           want_probs=False) -> SampleResult:
    a, pa = _f32(logits)
    h, ph = _i32(history)
    hc = 0 if h is None else h.size
    bi = bv = pbi = pbv = None
    nb = 0
    if bias:
        bi, pbi = _i32(list(bias.keys()))
        bv, pbv = _f32(list(bias.values()))
        nb = bi.size
    tr = OrcTrace()
    k = max(int(params.top_k), 1)
    cid = np.full(k, -1, np.int32)
    cv = np.zeros(k, np.float32)
    cp = np.zeros(k, np.float32)
    probs = np.zeros(a.size, np.float32) if want_probs else None
    tok = lib().orc_sample(
        pa, a.size, C.byref(params), ph, hc, pbi, pbv, nb, sum_mode, float(u), C.byref(tr),
        cid.ctypes.data_as(C.POINTER(C.c_int32)), cv.ctypes.data_as(C.POINTER(C.c_float)),
        cp.ctypes.data_as(C.POINTER(C.c_float)),
        probs.ctypes.data_as(C.POINTER(C.c_float)) if want_probs else None)
    return SampleResult(tok, tr, cid, cv, cp, probs)


def sample_bias_arrays(logits, params: OrcParams, u, history, bias_ids, bias_vals, sum_mode=0) -> SampleResult:
    """``sample`` with the logit bias given as parallel arrays (duplicate ids are added one after the
    other, as the reference's loop over the dictionary entries would for distinct keys)."""
    a, pa = _f32(logits)
    h, ph = _i32(history)
    hc = 0 if h is None else h.size
    bi, pbi = _i32(bias_ids)
    bv, pbv = _f32(bias_vals)
    tr = OrcTrace()
    k = max(int(params.top_k), 1)
    cid = np.full(k, -1, np.int32)
    cv = np.zeros(k, np.float32)
    cp = np.zeros(k, np.float32)
    tok = lib().orc_sample(
        pa, a.size, C.byref(params), ph, hc, pbi, pbv, bi.size, sum_mode, float(u), C.byref(tr),
        cid.ctypes.data_as(C.POINTER(C.c_int32)), cv.ctypes.data_as(C.POINTER(C.c_float)),
        cp.ctypes.data_as(C.POINTER(C.c_float)), None)
    return SampleResult(tok, tr, cid, cv, cp, None)


def build_filtered_distribution(logits, params: OrcParams, history=None, bias=None, sum_mode=0):
    a, pa = _f32(logits)
    h, ph = _i32(history)
    hc = 0 if h is None else h.size
    pbi = pbv = None
    nb = 0
    if bias:
        bi, pbi = _i32(list(bias.keys()))
        bv, pbv = _f32(list(bias.values()))
        nb = bi.size
    out = np.zeros(a.size, np.float32)
    tie = C.c_int32(0)
    lib().orc_build_filtered_distribution(pa, a.size, C.byref(params), ph, hc, pbi, pbv, nb,
                                          sum_mode, out.ctypes.data_as(C.POINTER(C.c_float)),
                                          C.byref(tie))
    return out, int(tie.value)


def build_filtered_distribution_ex(logits, params: OrcParams, history=None, bias_ids=None, bias_vals=None,
                                   sum_mode=0):
    """BuildFilteredDistribution with the bias as parallel arrays; returns (probs, tie, cut_margin):
    cut_margin is how close the sorted running sum of top-p came to top_p at the cut (inf: no top-p)."""
    a, pa = _f32(logits)
    h, ph = _i32(history)
    hc = 0 if h is None else h.size
    pbi = pbv = None
    nb = 0
    if bias_ids is not None and len(bias_ids):
        bi, pbi = _i32(bias_ids)
        bv, pbv = _f32(bias_vals)
        nb = bi.size
    out = np.zeros(a.size, np.float32)
    tie = C.c_int32(0)
    cm = C.c_float(0)
    lib().orc_build_filtered_distribution_ex(pa, a.size, C.byref(params), ph, hc, pbi, pbv, nb, sum_mode,
                                             out.ctypes.data_as(C.POINTER(C.c_float)), C.byref(tie), C.byref(cm))
    return out, int(tie.value), float(cm.value)


def sample_with_distribution(logits, params: OrcParams, u: float, history=None, sum_mode=0):
    a, pa = _f32(logits)
    h, ph = _i32(history)
    hc = 0 if h is None else h.size
    out = np.zeros(a.size, np.float32)
    tr = OrcTrace()
    tok = lib().orc_sample_with_distribution(pa, a.size, C.byref(params), ph, hc, sum_mode,
                                             float(u), out.ctypes.data_as(C.POINTER(C.c_float)),
                                             C.byref(tr))
    return tok, out, tr


def sample_from_probs(probs, u: float):
    a, pa = _f32(probs)
    tr = OrcTrace()
    return lib().orc_sample_from_probs(pa, a.size, float(u), C.byref(tr)), tr


def resample_residual(p, q, u0: float, u1: float = 0.5):
    a, pa = _f32(p)
    b, pb = _f32(q)
    if a.size != b.size:
        # ResampleResidual, Sampler.cs:590-592
        raise ValueError(f"p and q must have equal length ({a.size} vs {b.size}).")
    us = (C.c_double * 2)(u0, u1)
    used = C.c_int32(0)
    tr = OrcTrace()
    tok = lib().orc_resample_residual(pa, pb, a.size, us, C.byref(used), C.byref(tr))
    return tok, int(used.value), tr


def spec_step_sampled(target_rows, draft_rows, draft_tokens, params: OrcParams, u_accept, u_final,
                      mode=0, p_min=1.0, sum_mode=0):
    t, pt = _f32(target_rows)
    d, pd = _f32(draft_rows)
    tok, ptok = _i32(draft_tokens)
    n_draft = tok.size
    n = t.shape[-1]
    assert t.shape[0] == n_draft + 1
    ua = (C.c_double * max(n_draft, 1))(*[float(x) for x in u_accept])
    uf = (C.c_double * 2)(*[float(x) for x in u_final])
    corr = C.c_int32(-1)
    ap = np.zeros(max(n_draft, 1), np.float32)
    tr = OrcTrace()
    acc = lib().orc_spec_step_sampled(pt, pd, n, n_draft, ptok, C.byref(params), sum_mode, ua, uf,
                                      mode, float(p_min), C.byref(corr),
                                      ap.ctypes.data_as(C.POINTER(C.c_float)), C.byref(tr))
    return acc, int(corr.value), ap[:n_draft], tr


def spec_greedy_accept(rows, draft_tokens) -> int:
    t, pt = _f32(rows)
    tok, ptok = _i32(draft_tokens)
    return lib().orc_spec_greedy_accept(pt, t.shape[-1], tok.size, ptok)


def softmax_prob_at(logits, idx: int) -> float:
    a, pa = _f32(logits)
    return float(lib().orc_softmax_prob_at(pa, a.size, idx))


def mtp_accept(logits, draft: int, p_min: float):
    a, pa = _f32(logits)
    pr = C.c_float(0)
    ok = lib().orc_mtp_accept(pa, a.size, draft, float(p_min), C.byref(pr))
    return bool(ok), float(pr.value)


def apply_mask(logits, mask_words):
    a = np.array(logits, dtype=np.float32, copy=True)
    m = np.ascontiguousarray(mask_words, dtype=np.uint32)
    lib().orc_apply_mask(a.ctypes.data_as(C.POINTER(C.c_float)), a.size,
                         m.ctypes.data_as(C.POINTER(C.c_uint32)))
    return a


def and_masks(masks, n):
    ms = [np.ascontiguousarray(m, dtype=np.uint32) for m in masks]
    arr = (C.POINTER(C.c_uint32) * len(ms))(*[m.ctypes.data_as(C.POINTER(C.c_uint32)) for m in ms])
    out = np.zeros((n + 31) // 32, np.uint32)
    masking = lib().orc_and_masks(arr, len(ms), n, out.ctypes.data_as(C.POINTER(C.c_uint32)))
    return out, bool(masking)


def apply_history_penalties(logits, params: OrcParams, history):
    a = np.array(logits, dtype=np.float32, copy=True)
    h, ph = _i32(history)
    lib().orc_apply_history_penalties(a.ctypes.data_as(C.POINTER(C.c_float)), a.size,
                                      C.byref(params), ph, h.size)
    return a


def sample_rows(logits, params_arr, uniforms, hist_ids=None, hist_offsets=None, mask=None,
                sum_mode=0):
    """Serial per-row loop (ContinuousBatchingEngine.cs:609-644) over a [rows, n] array.

    ``logits`` is float32 or uint16 (bf16 bit patterns); ``params_arr`` a structured array of
    ``PARAMS_DTYPE``; ``uniforms`` one NextDouble() value per row.
    """
    logits = np.ascontiguousarray(logits)
    rows, n = logits.shape
    bf16 = logits.dtype == np.uint16
    assert bf16 or logits.dtype == np.float32
    params_arr = np.ascontiguousarray(params_arr, dtype=PARAMS_DTYPE)
    u = np.ascontiguousarray(uniforms, dtype=np.float64)
    tokens = np.zeros(rows, np.int32)
    traces = np.zeros(rows, TRACE_DTYPE)
    hi = ho = pm = None
    if hist_ids is not None:
        hi = np.ascontiguousarray(hist_ids, dtype=np.int32)
        ho = np.ascontiguousarray(hist_offsets, dtype=np.int32)
    mstride = 0
    if mask is not None:
        pm = np.ascontiguousarray(mask, dtype=np.uint32)
        mstride = pm.shape[1]
    lib().orc_sample_rows(
        logits.ctypes.data, int(bf16), rows, n, n, params_arr.ctypes.data,
        hi.ctypes.data_as(C.POINTER(C.c_int32)) if hi is not None else None,
        ho.ctypes.data_as(C.POINTER(C.c_int32)) if ho is not None else None,
        pm.ctypes.data_as(C.POINTER(C.c_uint32)) if pm is not None else None, mstride,
        u.ctypes.data_as(C.POINTER(C.c_double)), sum_mode,
        tokens.ctypes.data_as(C.POINTER(C.c_int32)), traces.ctypes.data)
    return tokens, traces
