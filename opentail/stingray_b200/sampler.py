"""Host-side mirror of the reference's sampler API over the C-ABI CUDA library.

Names, argument meaning and error behaviour follow the reference's managed API
(``src/OpenTail.Stingray.Engine/Sampler.cs``): ``SamplingParams`` keeps the reference's property
names, ``Sampler.Sample / Greedy / BuildFilteredDistribution / SampleWithDistribution`` keep their
signatures, and a ``Random`` is consumed exactly as there (one ``NextDouble()`` per non-greedy
sample, none when greedy).  ``BatchSampler`` is the batched form the reference does not have: one
call per decode step over device-resident ``[rows, vocab]`` logits, replacing the serial per-row
loop of ``ContinuousBatchingEngine.cs:609-644``.

Nothing here computes on the CPU: every method forwards to ``libstingray_sampler.so`` and raises
``StingrayError`` (the counterpart of the reference's ``InvalidOperationException`` on a non-zero
native status, ``CudaBackend.cs:4110-4111``) when the library reports a failure.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _native as N

PARAMS_DTYPE = np.dtype([
    ("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("repetition_penalty", "<f4"),
    ("presence_penalty", "<f4"), ("frequency_penalty", "<f4"), ("top_k", "<i4"),
    ("repeat_last_n", "<i4"),
])


class StingrayError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{N.ERR_NAMES.get(code, code)}: {message}")
        self.code = code


@dataclass
class SamplingParams:
    """The sampler-relevant fields of the reference's ``SamplingParams`` record
    (``Sampler.cs:648-686, 795``), same names and defaults."""

    Temperature: float = 1.0
    TopK: int = 0
    TopP: float = 1.0
    MinP: float = 0.0
    RepetitionPenalty: float = 1.0
    RepeatLastN: int = 64
    PresencePenalty: float = 0.0
    FrequencyPenalty: float = 0.0
    LogitBias: Optional[Dict[int, float]] = None
    PreviousTokens: Optional[Sequence[int]] = None
    SpecDraftPMin: float = 1.0

    @property
    def HasHistoryPenalty(self) -> bool:  # Sampler.cs:686
        return (np.float32(self.RepetitionPenalty) != 1.0 or np.float32(self.PresencePenalty) != 0.0
                or np.float32(self.FrequencyPenalty) != 0.0)

    def row(self):
        return (self.Temperature, self.TopP, self.MinP, self.RepetitionPenalty, self.PresencePenalty,
                self.FrequencyPenalty, self.TopK, self.RepeatLastN)


class Random:
    """Stand-in for ``System.Random``: only ``NextDouble()`` is used by the sampler.  The stream is
    NumPy's PCG64, not .NET's generator; what matters for parity is how many draws are consumed."""

    def __init__(self, seed: Optional[int] = None):
        self._g = np.random.default_rng(seed)
        self.draws = 0

    def NextDouble(self) -> float:
        self.draws += 1
        return float(self._g.random())


def _is_torch(x) -> bool:
    return hasattr(x, "data_ptr")


def _ptr(x) -> Optional[int]:
    if x is None:
        return None
    if _is_torch(x):
        return x.data_ptr()
    return x.ctypes.data


def params_array(params) -> np.ndarray:
    if isinstance(params, np.ndarray) and params.dtype == PARAMS_DTYPE:
        return np.ascontiguousarray(params)
    return np.array([p.row() for p in params], dtype=PARAMS_DTYPE)


class BatchSampler:
    """A library handle plus its workspace (``stg_create``).  One instance per device and calling
    thread, like the reference's backend (``IThreadAffineBackend.cs:11-21``)."""

    def __init__(self, max_rows: int, max_vocab: int, max_history: int = 512, max_top_k: int = 256,
                 max_bias: int = 64, max_spec_draft: int = 0, device: int = 0, host_logits: bool = False,
                 max_cached_masks: int = 0):
        """``host_logits``: reserve the device staging for host-resident logits and masks at creation
        (``STG_CFG_HOST_LOGITS``), so that no sampling call allocates.  ``max_cached_masks``: entries
        of the device-resident bitmask cache (``mask_cache_put`` / ``mask_compose``)."""
        self._lib = N.load()
        cfg = N.StgConfig(C.sizeof(N.StgConfig), device, max_rows, max_vocab, max_history, max_top_k,
                          max_bias, max_spec_draft, N.CFG_HOST_LOGITS if host_logits else 0, max_cached_masks)
        h = C.c_void_p()
        rc = self._lib.stg_create(C.byref(cfg), C.byref(h))
        if rc != N.STG_OK:
            raise StingrayError(rc, self._error(None))
        self._h = h
        self.device = device
        self.max_rows, self.max_vocab, self.max_top_k = max_rows, max_vocab, max_top_k

    # -- plumbing -------------------------------------------------------------------------------
    def _error(self, h) -> str:
        buf = C.create_string_buffer(512)
        self._lib.stg_last_error(h, buf, 512)
        return buf.value.decode("utf-8", "replace")

    def _check(self, rc: int):
        if rc != N.STG_OK:
            raise StingrayError(rc, self._error(self._h))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.stg_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def stats(self) -> dict:
        s = N.StgStats()
        self._check(self._lib.stg_get_stats(self._h, C.byref(s)))
        return {n: getattr(s, n) for n, _ in s._fields_}

    @staticmethod
    def _stream(stream) -> Optional[int]:
        if stream is not None:
            return getattr(stream, "cuda_stream", stream)  # a torch.cuda.Stream or a raw handle
        import torch

        return torch.cuda.current_stream().cuda_stream

    def _alloc(self, shape, dtype, host: bool):
        if host:
            return np.empty(shape, dtype)
        import torch

        td = {np.int32: torch.int32, np.float32: torch.float32, np.uint32: torch.int32}[dtype]
        return torch.empty(shape, dtype=td, device=f"cuda:{self.device}")

    def _batch(self, logits, params, history_ids, history_offsets, mask, row_uses_mask, bias,
               uniforms, softcap: float = 0.0, history_ring: bool = False):
        """Builds the StgSampleBatch; returns it with the objects that must stay alive."""
        keep = []
        rows, vocab = logits.shape
        if _is_torch(logits):
            import torch

            assert logits.is_cuda and logits.stride(1) == 1
            dtype = {torch.float32: N.DTYPE_F32, torch.bfloat16: N.DTYPE_BF16}[logits.dtype]
            stride = logits.stride(0) if rows > 1 else vocab
            flags = 0
        else:
            logits = np.ascontiguousarray(logits)
            dtype = N.DTYPE_BF16 if logits.dtype == np.uint16 else N.DTYPE_F32
            assert logits.dtype in (np.float32, np.uint16)
            stride = vocab
            flags = N.MEM_HOST_LOGITS
        keep.append(logits)
        pa = params_array(params)
        assert pa.shape[0] == rows
        keep.append(pa)
        b = N.StgSampleBatch()
        b.struct_size = C.sizeof(N.StgSampleBatch)
        b.rows, b.vocab, b.logits_dtype = rows, vocab, dtype
        b.logits, b.row_stride, b.params = _ptr(logits), stride, pa.ctypes.data
        if history_ring:
            assert history_ids is None, "history_ring uses the handle's own histories"
            flags |= N.MEM_HISTORY_RING
        elif history_ids is not None:
            ho = np.ascontiguousarray(history_offsets, dtype=np.int32)
            if not _is_torch(history_ids):
                history_ids = np.ascontiguousarray(history_ids, dtype=np.int32)
                flags |= N.MEM_HOST_HISTORY
            keep += [ho, history_ids]
            b.history_ids, b.history_offsets = _ptr(history_ids), ho.ctypes.data
        if mask is not None:
            if not _is_torch(mask):
                mask = np.ascontiguousarray(mask, dtype=np.uint32)
                flags |= N.MEM_HOST_MASK
                mstride = mask.shape[1]
            else:
                mstride = mask.stride(0) if rows > 1 else mask.shape[1]
            keep.append(mask)
            b.mask, b.mask_row_stride = _ptr(mask), mstride
            if row_uses_mask is not None:
                rum = np.ascontiguousarray(row_uses_mask, dtype=np.uint8)
                keep.append(rum)
                b.row_uses_mask = rum.ctypes.data
        if bias is not None:
            bi, bv, bo = bias
            bo = np.ascontiguousarray(bo, dtype=np.int32)
            if not _is_torch(bi):
                bi = np.ascontiguousarray(bi, dtype=np.int32)
                bv = np.ascontiguousarray(bv, dtype=np.float32)
                flags |= N.MEM_HOST_BIAS
            keep += [bi, bv, bo]
            b.bias_ids, b.bias_values, b.bias_offsets = _ptr(bi), _ptr(bv), bo.ctypes.data
        if uniforms is not None:
            if not _is_torch(uniforms):
                uniforms = np.ascontiguousarray(uniforms, dtype=np.float32)
                flags |= N.MEM_HOST_UNIFORMS
            keep.append(uniforms)
            b.uniforms = _ptr(uniforms)
        b.mem_flags = flags
        b.logit_softcap = softcap
        return b, keep

    # -- entry points ------------------------------------------------------------------------------
    def argmax_rows(self, logits, valid_len: Optional[int] = None, stream=None):
        """``CudaBackend.ArgmaxRowsToDevice`` (``CudaBackend.cs:4176-4190``): returns device
        tensors (index, value) of the per-row argmax over ``[0, valid_len)``."""
        import torch

        rows, width = logits.shape
        vocab = width if valid_len is None else valid_len
        dtype = {torch.float32: N.DTYPE_F32, torch.bfloat16: N.DTYPE_BF16}[logits.dtype]
        out = torch.empty((rows, 2), dtype=torch.int32, device=logits.device)
        self._check(self._lib.stg_argmax_rows(self._h, logits.data_ptr(), dtype, rows, vocab,
                                              logits.stride(0) if rows > 1 else width,
                                              out.data_ptr(), self._stream(stream)))
        return out[:, 0], out[:, 1].view(torch.float32)

    def sample_rows(self, logits, params, *, history_ids=None, history_offsets=None, mask=None,
                    row_uses_mask=None, bias=None, uniforms=None, want_probs=False,
                    want_flags=False, want_topk=0, host_outputs: Optional[bool] = None, softcap: float = 0.0,
                    history_ring: bool = False, stream=None, out: Optional[dict] = None):
        """One sampling step (``stg_sample_rows``).  ``logits`` is a CUDA tensor (fp32/bf16) or a
        NumPy array (float32, or uint16 bf16 bit patterns); ``params`` a list of SamplingParams or
        a PARAMS_DTYPE array; histories/bias are CSR; ``uniforms`` one float per row.  Returns a
        dict with ``tokens`` and the optional outputs, on the device unless ``host_outputs``.
        ``softcap`` != 0 reads every logit as ``tanh(x / softcap) * softcap`` (the final-logit soft
        cap, ``CudaTextKernels.cs:374-383``) without rewriting the logits.  ``history_ring``: row r's
        PreviousTokens are the handle's device-resident history of slot r (``history_append``).
        ``out``: the dict a previous call with the same shapes and options returned; its arrays are
        written again instead of new ones (a decode loop's fixed output buffers - with the inputs in
        place too, the step repeats exactly and the library replays it as a CUDA graph)."""
        b, keep = self._batch(logits, params, history_ids, history_offsets, mask, row_uses_mask,
                              bias, uniforms, softcap, history_ring)
        host = (not _is_torch(logits)) if host_outputs is None else host_outputs
        rows = b.rows
        prev = out

        def take(name, shape, dtype):
            if prev is not None:
                arr = prev[name]
                if tuple(arr.shape) != tuple(shape):
                    raise ValueError(f"out[{name!r}] has shape {tuple(arr.shape)}, this call needs {tuple(shape)}")
                return arr
            return self._alloc(shape, dtype, host)

        out = {"tokens": take("tokens", (rows,), np.int32)}
        b.tokens = _ptr(out["tokens"])
        if want_probs:
            out["probs"] = take("probs", (rows,), np.float32)
            b.token_probs = _ptr(out["probs"])
        if want_flags:
            out["flags"] = take("flags", (rows,), np.uint32)
            b.row_flags = _ptr(out["flags"])
        if want_topk:
            out["topk_ids"] = take("topk_ids", (rows, want_topk), np.int32)
            out["topk_logits"] = take("topk_logits", (rows, want_topk), np.float32)
            out["topk_probs"] = take("topk_probs", (rows, want_topk), np.float32)
            b.topk_ids, b.topk_logits = _ptr(out["topk_ids"]), _ptr(out["topk_logits"])
            b.topk_probs, b.topk_stride = _ptr(out["topk_probs"]), want_topk
        if host:
            b.mem_flags |= N.MEM_HOST_OUTPUTS
        self._check(self._lib.stg_sample_rows(self._h, C.byref(b), self._stream(stream)))
        return out

    def build_distribution(self, logits, params, *, history_ids=None, history_offsets=None,
                           mask=None, bias=None, host_outputs: Optional[bool] = None, softcap: float = 0.0,
                           stream=None):
        """``Sampler.BuildFilteredDistribution`` for every row: returns ``[rows, vocab]`` float32."""
        b, keep = self._batch(logits, params, history_ids, history_offsets, mask, None, bias, None, softcap)
        host = (not _is_torch(logits)) if host_outputs is None else host_outputs
        probs = self._alloc((b.rows, b.vocab), np.float32, host)
        if host:
            b.mem_flags |= N.MEM_HOST_OUTPUTS
        self._check(self._lib.stg_build_distribution(self._h, C.byref(b), _ptr(probs),
                                                     self._stream(stream)))
        return probs

    def sample_with_distribution(self, logits, params, *, history_ids=None, history_offsets=None, mask=None,
                                 uniforms=None, want_probs=True, softcap: float = 0.0, stream=None):
        """``Sampler.SampleWithDistribution`` for every row (``stg_sample_with_distribution``): the
        full-vocabulary pipeline whatever ``TopK`` is.  ``logits`` is a CUDA tensor; returns
        (tokens, probs ``[rows, vocab]`` or None), both on the device."""
        b, keep = self._batch(logits, params, history_ids, history_offsets, mask, None, None, uniforms, softcap)
        tokens = self._alloc((b.rows,), np.int32, False)
        b.tokens = _ptr(tokens)
        probs = self._alloc((b.rows, b.vocab), np.float32, False) if want_probs else None
        self._check(self._lib.stg_sample_with_distribution(self._h, C.byref(b), _ptr(probs), self._stream(stream)))
        return tokens, probs

    def sample_from_probs(self, probs, uniforms, stream=None):
        """``Sampler.SampleFromProbs`` per row of a CUDA ``[rows, vocab]`` float32 tensor."""
        import torch

        rows, vocab = probs.shape
        assert probs.is_cuda and probs.dtype == torch.float32 and probs.stride(1) == 1
        flags = 0
        if not _is_torch(uniforms):
            uniforms = np.ascontiguousarray(uniforms, dtype=np.float32)
            flags |= N.MEM_HOST_UNIFORMS
        tokens = self._alloc((rows,), np.int32, False)
        rf = self._alloc((rows,), np.uint32, False)
        self._check(self._lib.stg_sample_from_probs(self._h, probs.data_ptr(), rows, vocab, probs.stride(0) if rows > 1 else vocab,
                                                    _ptr(uniforms), _ptr(tokens), _ptr(rf), flags, self._stream(stream)))
        return tokens, rf

    def resample_residual(self, p, q, uniforms, stream=None):
        """``Sampler.ResampleResidual`` per row; ``p`` and ``q`` CUDA ``[rows, vocab]`` float32 tensors of
        equal shape, ``uniforms`` ``[rows, 2]``."""
        import torch

        if tuple(p.shape) != tuple(q.shape):
            # ResampleResidual, Sampler.cs:590-592
            raise ValueError(f"p and q must have equal length ({p.shape[-1]} vs {q.shape[-1]}).")
        rows, vocab = p.shape
        assert p.is_cuda and q.is_cuda and p.dtype == torch.float32 and q.dtype == torch.float32
        assert p.stride(1) == 1 and q.stride() == p.stride()
        flags = 0
        if not _is_torch(uniforms):
            uniforms = np.ascontiguousarray(uniforms, dtype=np.float32).reshape(rows, 2)
            flags |= N.MEM_HOST_UNIFORMS
        tokens = self._alloc((rows,), np.int32, False)
        rf = self._alloc((rows,), np.uint32, False)
        self._check(self._lib.stg_resample_residual(self._h, p.data_ptr(), q.data_ptr(), rows, vocab,
                                                    p.stride(0) if rows > 1 else vocab, _ptr(uniforms), _ptr(tokens),
                                                    _ptr(rf), flags, self._stream(stream)))
        return tokens, rf

    def spec_verify(self, target_logits, draft_logits, draft_tokens, params, uniforms, *, mode=0,
                    p_min=1.0, want_probs=False, target_softcap: float = 0.0, draft_softcap: float = 0.0,
                    stream=None):
        """``SpeculativeDecoder.StepSampled``'s accept loop for ``n_seq`` sequences
        (``stg_spec_verify``).  target ``[n_seq, L + 1, V]``, draft ``[n_seq, L, V]`` CUDA tensors,
        draft_tokens ``[n_seq, L]`` int32, uniforms ``[n_seq, L + 2]`` float64 (host or device)."""
        import torch

        n_seq, lp1, vocab = target_logits.shape
        L = lp1 - 1
        pa = params_array(params)
        dtype = {torch.float32: N.DTYPE_F32, torch.bfloat16: N.DTYPE_BF16}[target_logits.dtype]
        flags = 0
        if not _is_torch(draft_tokens):
            draft_tokens = np.ascontiguousarray(draft_tokens, dtype=np.int32)
            flags |= N.MEM_HOST_DRAFT
        if not _is_torch(uniforms):
            uniforms = np.ascontiguousarray(uniforms, dtype=np.float64)
            flags |= N.MEM_HOST_UNIFORMS
        dev = target_logits.device
        accepted = torch.empty(n_seq, dtype=torch.int32, device=dev)
        correction = torch.empty(n_seq, dtype=torch.int32, device=dev)
        aprobs = torch.empty((n_seq, max(L, 1)), dtype=torch.float32, device=dev)
        sflags = torch.empty(n_seq, dtype=torch.int32, device=dev)
        b = N.StgSpecBatch()
        b.struct_size = C.sizeof(N.StgSpecBatch)
        b.n_seq, b.n_draft, b.vocab, b.logits_dtype, b.mode = n_seq, L, vocab, dtype, mode
        assert target_logits.is_contiguous() and (draft_logits is None or draft_logits.is_contiguous())
        b.target_logits = target_logits.data_ptr()
        b.draft_logits = draft_logits.data_ptr() if draft_logits is not None else None
        b.draft_tokens, b.params, b.uniforms = _ptr(draft_tokens), pa.ctypes.data, _ptr(uniforms)
        b.p_min = p_min
        b.target_softcap, b.draft_softcap = target_softcap, draft_softcap
        b.accepted, b.correction = accepted.data_ptr(), correction.data_ptr()
        b.accept_probs, b.seq_flags, b.mem_flags = aprobs.data_ptr(), sflags.data_ptr(), flags
        self._check(self._lib.stg_spec_verify(self._h, C.byref(b), self._stream(stream)))
        out = {"accepted": accepted, "correction": correction, "flags": sflags}
        if want_probs:
            out["accept_probs"] = aprobs
        return out

    def mtp_accept(self, logits, draft_tokens, p_min: float, stream=None):
        """``MtpDecoder.AcceptDraft`` per row (``stg_mtp_accept``): returns (accept, argmax, prob)."""
        import torch

        rows, vocab = logits.shape
        dtype = {torch.float32: N.DTYPE_F32, torch.bfloat16: N.DTYPE_BF16}[logits.dtype]
        acc = torch.empty(rows, dtype=torch.int32, device=logits.device)
        am = torch.empty(rows, dtype=torch.int32, device=logits.device)
        pr = torch.empty(rows, dtype=torch.float32, device=logits.device)
        self._check(self._lib.stg_mtp_accept(self._h, logits.data_ptr(), dtype, rows, vocab,
                                             logits.stride(0) if rows > 1 else vocab,
                                             draft_tokens.data_ptr(), p_min, acc.data_ptr(),
                                             am.data_ptr(), pr.data_ptr(), self._stream(stream)))
        return acc, am, pr

    def and_masks(self, masks, vocab: int, stream=None):
        """``AndTokenConstraint.Filter`` in bitmask form (``stg_and_masks``): ``masks`` is a CUDA int32
        tensor ``[n_masks, rows, words]`` of allowed-token bits; returns (mask ``[rows, words]``,
        uses ``[rows]`` uint8: 0 where the row comes out unmasked)."""
        import torch

        n_masks, rows, words = masks.shape
        assert masks.is_contiguous() and masks.dtype == torch.int32
        out = torch.empty((rows, words), dtype=torch.int32, device=masks.device)
        uses = torch.empty(rows, dtype=torch.uint8, device=masks.device)
        self._check(self._lib.stg_and_masks(self._h, C.c_void_p(masks.data_ptr()), n_masks, rows, vocab,
                                            C.c_int64(words), C.c_void_p(out.data_ptr()), C.c_int64(words),
                                            C.c_void_p(uses.data_ptr()), self._stream(stream)))
        return out, uses

    # -- bitmask cache ---------------------------------------------------------------------------------
    def mask_cache_put(self, key: int, words, vocab: int, stream=None):
        """Stores a host bitmask (uint32 words) under ``key`` (``stg_mask_cache_put``)."""
        w = np.ascontiguousarray(words, dtype=np.uint32)
        assert w.size >= (vocab + 31) // 32
        self._check(self._lib.stg_mask_cache_put(self._h, C.c_uint64(key), w.ctypes.data, vocab, self._stream(stream)))

    def mask_cache_contains(self, key: int) -> bool:
        return bool(self._lib.stg_mask_cache_contains(self._h, C.c_uint64(key)))

    def mask_cache_get_or_put(self, key: int, vocab: int, allowed_tokens, stream=None) -> bool:
        """The use the cache is made for: ``allowed_tokens()`` - the walk over the vocabulary that
        ``JsonSchemaGrammarMasker.Filter`` (``JsonSchemaGrammarMasker.cs:67-95``) repeats every step -
        is called only when the (constraint, state) ``key`` has not been seen; it returns the ids of
        the allowed tokens.  Returns True when the walk ran."""
        if self.mask_cache_contains(key):
            return False
        words = np.zeros((vocab + 31) // 32, dtype=np.uint32)
        ids = np.asarray(allowed_tokens(), dtype=np.int64)
        np.bitwise_or.at(words, ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
        self.mask_cache_put(key, words, vocab, stream)
        return True

    def mask_compose(self, keys, vocab: int, op: str = "and", stream=None):
        """``stg_mask_compose``: ``keys`` is ``[rows, keys_per_row]`` (0 = empty slot); returns the
        device mask ``[rows, words]`` (int32 view of the words) and the per-row uses-mask bytes."""
        import torch

        k = np.ascontiguousarray(keys, dtype=np.uint64)
        rows, per = k.shape
        words = (vocab + 31) // 32
        dev = f"cuda:{self.device}"
        out = torch.empty((rows, words), dtype=torch.int32, device=dev)
        uses = torch.empty(rows, dtype=torch.uint8, device=dev)
        self._check(self._lib.stg_mask_compose(self._h, k.ctypes.data, per, rows, vocab,
                                               {"and": N.MASK_AND, "or": N.MASK_OR}[op], C.c_void_p(out.data_ptr()),
                                               C.c_int64(words), C.c_void_p(uses.data_ptr()), self._stream(stream)))
        return out, uses

    # -- device-resident histories ---------------------------------------------------------------------
    def history_reset(self, first_slot: int = 0, n_slots: Optional[int] = None, stream=None):
        n = self.max_rows - first_slot if n_slots is None else n_slots
        self._check(self._lib.stg_history_reset(self._h, first_slot, n, self._stream(stream)))

    def history_load(self, slot: int, tokens, stream=None):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        self._check(self._lib.stg_history_load(self._h, slot, t.ctypes.data, t.size, self._stream(stream)))

    def history_append(self, tokens, active=None, stream=None):
        """Appends ``tokens[r]`` (device int32 tensor, e.g. the ``tokens`` a step returned) to slot r."""
        assert _is_torch(tokens) and tokens.is_cuda
        act = None if active is None else np.ascontiguousarray(active, dtype=np.uint8)
        self._check(self._lib.stg_history_append(self._h, tokens.data_ptr(), tokens.numel(),
                                                 None if act is None else act.ctypes.data, self._stream(stream)))

    def history_length(self, slot: int) -> int:
        n = self._lib.stg_history_length(self._h, slot)
        if n < 0:
            raise StingrayError(-n, self._error(self._h))
        return n

    # -- vocabulary-sharded mode ---------------------------------------------------------------------
    @staticmethod
    def comm_unique_id() -> bytes:
        """128 bytes identifying a new communicator; create on rank 0 and broadcast."""
        buf = C.create_string_buffer(128)
        rc = N.load().stg_comm_unique_id(buf)
        if rc != N.STG_OK:
            raise StingrayError(rc, "stg_comm_unique_id failed")
        return buf.raw

    def comm_init(self, unique_id: bytes, rank: int, n_ranks: int):
        self._check(self._lib.stg_comm_init(self._h, unique_id, rank, n_ranks))

    def shard_select(self, logits, params, vocab_offset: int, global_vocab: int, *, history_ids=None,
                     history_offsets=None, mask=None, uniforms=None, stream=None):
        """Selects this rank's candidates over its vocabulary slice (``stg_shard_select``)."""
        b, keep = self._batch(logits, params, history_ids, history_offsets, mask, None, None, uniforms)
        self._check(self._lib.stg_shard_select(self._h, C.byref(b), vocab_offset, global_vocab,
                                               self._stream(stream)))

    def shard_allgather(self, stream=None):
        self._check(self._lib.stg_shard_allgather(self._h, self._stream(stream)))

    def exchange_bytes(self) -> int:
        """Bytes this rank sends in the all-gather of the step last selected."""
        n = C.c_uint64(0)
        self._check(self._lib.stg_shard_exchange_bytes(self._h, C.byref(n)))
        return int(n.value)

    def shard_gather_local(self, peers: "Sequence[BatchSampler]", stream=None):
        arr = (C.c_void_p * len(peers))(*[p._h for p in peers])
        self._check(self._lib.stg_shard_gather_local(self._h, arr, len(peers), self._stream(stream)))

    def shard_finish(self, rows: int, local_vocab: int, params, global_vocab: int, *, history_ids=None,
                     history_offsets=None, uniforms=None, want_probs=False, want_flags=False,
                     want_topk=0, stream=None):
        """Merges the gathered candidates and finishes every row (``stg_shard_finish``)."""
        import torch

        pa = params_array(params)
        b = N.StgSampleBatch()
        b.struct_size = C.sizeof(N.StgSampleBatch)
        b.rows, b.vocab, b.logits_dtype, b.row_stride = rows, local_vocab, N.DTYPE_F32, local_vocab
        b.params = pa.ctypes.data
        keep = [pa]
        flags = 0
        if history_ids is not None:
            ho = np.ascontiguousarray(history_offsets, dtype=np.int32)
            if not _is_torch(history_ids):
                history_ids = np.ascontiguousarray(history_ids, dtype=np.int32)
                flags |= N.MEM_HOST_HISTORY
            keep += [ho, history_ids]
            b.history_ids, b.history_offsets = _ptr(history_ids), ho.ctypes.data
        if uniforms is not None:
            if not _is_torch(uniforms):
                uniforms = np.ascontiguousarray(uniforms, dtype=np.float32)
                flags |= N.MEM_HOST_UNIFORMS
            keep.append(uniforms)
            b.uniforms = _ptr(uniforms)
        b.mem_flags = flags
        out = {"tokens": self._alloc((rows,), np.int32, False)}
        b.tokens = _ptr(out["tokens"])
        if want_probs:
            out["probs"] = self._alloc((rows,), np.float32, False)
            b.token_probs = _ptr(out["probs"])
        if want_flags:
            out["flags"] = self._alloc((rows,), np.uint32, False)
            b.row_flags = _ptr(out["flags"])
        if want_topk:
            out["topk_ids"] = self._alloc((rows, want_topk), np.int32, False)
            out["topk_logits"] = self._alloc((rows, want_topk), np.float32, False)
            out["topk_probs"] = self._alloc((rows, want_topk), np.float32, False)
            b.topk_ids, b.topk_logits = _ptr(out["topk_ids"]), _ptr(out["topk_logits"])
            b.topk_probs, b.topk_stride = _ptr(out["topk_probs"]), want_topk
        self._check(self._lib.stg_shard_finish(self._h, C.byref(b), global_vocab, self._stream(stream)))
        return out


_shared: Dict[int, BatchSampler] = {}


def _single(vocab: int) -> BatchSampler:
    """Handle used by the static single-row API, grown when a larger vocabulary shows up."""
    s = _shared.get(0)
    if s is None or s.max_vocab < vocab:
        if s is not None:
            s.close()
        s = BatchSampler(max_rows=8, max_vocab=max(vocab, 4096), max_history=4096, max_top_k=1024,
                         max_bias=256)
        _shared[0] = s
    return s


def _csr(seq):
    ids = np.asarray(list(seq) if seq is not None else [], dtype=np.int32)
    return ids, np.array([0, ids.size], dtype=np.int32)


class Sampler:
    """Static single-row API with the reference's signatures (``Sampler.cs:12-646``)."""

    @staticmethod
    def Greedy(logits) -> int:
        """``Sampler.Greedy`` (``Sampler.cs:442-446``): highest logit, lowest index on ties;
        an empty span returns 0."""
        a = np.ascontiguousarray(logits, dtype=np.float32).reshape(1, -1)
        if a.shape[1] == 0:
            return 0
        p = SamplingParams(Temperature=0.0)
        return int(_single(a.shape[1]).sample_rows(a, [p])["tokens"][0])

    @staticmethod
    def Sample(logits, p: SamplingParams, rng: Optional[Random] = None) -> int:
        """``Sampler.Sample`` (``Sampler.cs:17-102``)."""
        a = np.ascontiguousarray(logits, dtype=np.float32).reshape(1, -1)
        kw = {}
        if p.PreviousTokens is not None and len(p.PreviousTokens) > 0:
            kw["history_ids"], kw["history_offsets"] = _csr(p.PreviousTokens)
        if p.Temperature > 0:
            rng = rng or _default_rng
            kw["uniforms"] = np.array([np.float32(rng.NextDouble())], dtype=np.float32)
            if p.LogitBias:
                ids = np.array(list(p.LogitBias.keys()), dtype=np.int32)
                vals = np.array(list(p.LogitBias.values()), dtype=np.float32)
                kw["bias"] = (ids, vals, np.array([0, ids.size], dtype=np.int32))
        return int(_single(a.shape[1]).sample_rows(a, [p], **kw)["tokens"][0])

    @staticmethod
    def BuildFilteredDistribution(logits, p: SamplingParams, probs: np.ndarray) -> None:
        """``Sampler.BuildFilteredDistribution`` (``Sampler.cs:118-163``): fills ``probs``."""
        a = np.ascontiguousarray(logits, dtype=np.float32).reshape(1, -1)
        if probs.shape[-1] != a.shape[1]:
            raise ValueError(
                f"probs length ({probs.shape[-1]}) must equal logits length ({a.shape[1]}).")
        kw = {}
        if p.PreviousTokens is not None and len(p.PreviousTokens) > 0:
            kw["history_ids"], kw["history_offsets"] = _csr(p.PreviousTokens)
        if p.LogitBias and p.Temperature > 0:
            ids = np.array(list(p.LogitBias.keys()), dtype=np.int32)
            vals = np.array(list(p.LogitBias.values()), dtype=np.float32)
            kw["bias"] = (ids, vals, np.array([0, ids.size], dtype=np.int32))
        probs[...] = _single(a.shape[1]).build_distribution(a, [p], **kw)[0]


    @staticmethod
    def SampleWithDistribution(logits, p: SamplingParams, probs: np.ndarray, rng: Optional[Random] = None) -> int:
        """``Sampler.SampleWithDistribution`` (``Sampler.cs:172-187``): fills ``probs`` and returns the
        drawn token; one ``NextDouble()`` is consumed unless ``Temperature <= 0``."""
        import torch

        a = np.ascontiguousarray(logits, dtype=np.float32).reshape(1, -1)
        if probs.shape[-1] != a.shape[1]:
            raise ValueError(f"probs length ({probs.shape[-1]}) must equal logits length ({a.shape[1]}).")
        kw = {}
        if p.PreviousTokens is not None and len(p.PreviousTokens) > 0:
            ids, off = _csr(p.PreviousTokens)
            kw["history_ids"], kw["history_offsets"] = torch.from_numpy(ids).cuda(), off
        if p.Temperature > 0:
            rng = rng or _default_rng
            kw["uniforms"] = torch.tensor([np.float32(rng.NextDouble())], dtype=torch.float32, device="cuda")
        tok, pr = _single(a.shape[1]).sample_with_distribution(torch.from_numpy(a).cuda(), [p], **kw)
        probs[...] = pr[0].cpu().numpy()
        return int(tok[0].item())

    @staticmethod
    def SampleFromProbs(probs, rng: Random) -> int:
        """``Sampler.SampleFromProbs`` (``Sampler.cs:195-199``)."""
        import torch

        if rng is None:
            raise ValueError("rng must not be None")  # ArgumentNullException.ThrowIfNull(rng)
        a = np.ascontiguousarray(probs, dtype=np.float32).reshape(1, -1)
        u = np.array([np.float32(rng.NextDouble())], dtype=np.float32)
        tok, _ = _single(a.shape[1]).sample_from_probs(torch.from_numpy(a).cuda(), u)
        return int(tok[0].item())

    @staticmethod
    def ResampleResidual(p, q, rng: Random) -> int:
        """``Sampler.ResampleResidual`` (``Sampler.cs:587-618``).  One ``NextDouble()`` is consumed, as in
        the reference; its last-resort second draw (no positive residual although their sum was
        positive) cannot occur, and a fixed 0.5 stands in for it."""
        import torch

        if rng is None:
            raise ValueError("rng must not be None")
        pa = np.ascontiguousarray(p, dtype=np.float32).reshape(1, -1)
        qa = np.ascontiguousarray(q, dtype=np.float32).reshape(1, -1)
        if pa.shape != qa.shape:
            raise ValueError(f"p and q must have equal length ({pa.shape[1]} vs {qa.shape[1]}).")
        u = np.array([[np.float32(rng.NextDouble()), 0.5]], dtype=np.float32)
        tok, _ = _single(pa.shape[1]).resample_residual(torch.from_numpy(pa).cuda(), torch.from_numpy(qa).cuda(), u)
        return int(tok[0].item())


_default_rng = Random()
