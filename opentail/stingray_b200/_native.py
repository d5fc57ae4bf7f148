"""ctypes view of ``include/stingray_sampler.h`` (what a C# host binds with LibraryImport)."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libstingray_sampler.so")

STG_OK = 0
ERR_NAMES = {
    1: "STG_ERR_INVALID_ARGUMENT", 2: "STG_ERR_CUDA", 3: "STG_ERR_CAPACITY", 4: "STG_ERR_UNSUPPORTED",
    5: "STG_ERR_TIMEOUT", 6: "STG_ERR_NCCL", 7: "STG_ERR_NO_DEVICE",
}
DTYPE_F32, DTYPE_BF16 = 0, 1
MEM_HOST_LOGITS, MEM_HOST_HISTORY, MEM_HOST_MASK, MEM_HOST_BIAS = 1, 2, 4, 8
MEM_HOST_UNIFORMS, MEM_HOST_OUTPUTS, MEM_HOST_DRAFT = 16, 32, 64
MEM_HISTORY_RING = 128
MASK_AND, MASK_OR = 0, 1
CFG_HOST_LOGITS = 1
SEQ_EMPTY_RESIDUAL, SEQ_BAD_DRAFT = 1 << 8, 1 << 9

EXPORTS = [
    "stg_abi_version", "stg_create", "stg_destroy", "stg_last_error", "stg_get_stats", "stg_debug_phase_ticks",
    "stg_debug_kernel_times", "stg_debug_check_guards",
    "stg_argmax_rows", "stg_argmax_rows_static", "stg_sample_rows", "stg_build_distribution", "stg_spec_verify",
    "stg_sample_with_distribution", "stg_sample_from_probs", "stg_resample_residual",
    "stg_mtp_accept", "stg_and_masks", "stg_comm_unique_id", "stg_comm_init", "stg_comm_destroy",
    "stg_shard_select", "stg_shard_allgather", "stg_shard_exchange_bytes", "stg_shard_finish", "stg_shard_gather_local",
    "stg_mask_cache_put", "stg_mask_cache_contains", "stg_mask_compose",
    "stg_history_reset", "stg_history_load", "stg_history_append", "stg_history_length",
]


class StgConfig(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("device", C.c_int32), ("max_rows", C.c_int32),
        ("max_vocab", C.c_int32), ("max_history", C.c_int32), ("max_top_k", C.c_int32),
        ("max_bias", C.c_int32), ("max_spec_draft", C.c_int32), ("flags", C.c_uint32),
        ("max_cached_masks", C.c_int32),
    ]


class StgRowParams(C.Structure):
    _fields_ = [
        ("temperature", C.c_float), ("top_p", C.c_float), ("min_p", C.c_float),
        ("repetition_penalty", C.c_float), ("presence_penalty", C.c_float),
        ("frequency_penalty", C.c_float), ("top_k", C.c_int32), ("repeat_last_n", C.c_int32),
    ]


class StgSampleBatch(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("rows", C.c_int32), ("vocab", C.c_int32),
        ("logits_dtype", C.c_int32), ("logits", C.c_void_p), ("row_stride", C.c_int64),
        ("params", C.c_void_p), ("history_ids", C.c_void_p), ("history_offsets", C.c_void_p),
        ("mask", C.c_void_p), ("mask_row_stride", C.c_int64), ("row_uses_mask", C.c_void_p),
        ("bias_ids", C.c_void_p), ("bias_values", C.c_void_p), ("bias_offsets", C.c_void_p),
        ("uniforms", C.c_void_p), ("tokens", C.c_void_p), ("token_probs", C.c_void_p),
        ("row_flags", C.c_void_p), ("topk_ids", C.c_void_p), ("topk_logits", C.c_void_p),
        ("topk_probs", C.c_void_p), ("topk_stride", C.c_int32), ("mem_flags", C.c_uint32),
        ("logit_softcap", C.c_float),
    ]


class StgSpecBatch(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("n_seq", C.c_int32), ("n_draft", C.c_int32),
        ("vocab", C.c_int32), ("logits_dtype", C.c_int32), ("mode", C.c_int32),
        ("target_logits", C.c_void_p), ("draft_logits", C.c_void_p), ("draft_tokens", C.c_void_p),
        ("params", C.c_void_p), ("uniforms", C.c_void_p), ("p_min", C.c_float),
        ("accepted", C.c_void_p), ("correction", C.c_void_p), ("accept_probs", C.c_void_p),
        ("seq_flags", C.c_void_p), ("mem_flags", C.c_uint32),
        ("target_softcap", C.c_float), ("draft_softcap", C.c_float),
    ]


class StgStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "calls", "rows_sampled", "rows_greedy", "rows_topk_path", "rows_full_path",
        "sequences_verified", "kernel_launches", "plan_uploads", "boundary_draws", "tie_rows", "cdf_fallbacks",
        "wide_nucleus_rows", "reread_rows", "near_cut_rows", "fully_masked_rows", "graph_replays")]


_lib = None


def load() -> C.CDLL:
    """Loads the CUDA library; raises (never substitutes a CPU path) when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m opentail.stingray_b200.build`. "
            "There is no CPU fallback for the sampling path.")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
    lib.stg_abi_version.restype = C.c_int
    lib.stg_create.argtypes = [C.POINTER(StgConfig), C.POINTER(vp)]
    lib.stg_destroy.argtypes = [vp]
    lib.stg_last_error.restype = C.c_size_t
    lib.stg_last_error.argtypes = [vp, C.c_char_p, C.c_size_t]
    lib.stg_get_stats.argtypes = [vp, C.POINTER(StgStats)]
    lib.stg_debug_phase_ticks.argtypes = [vp, vp, i32, C.POINTER(C.c_int32)]
    lib.stg_debug_check_guards.argtypes = [vp, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.stg_debug_kernel_times.argtypes = [vp, vp, vp, i32, i32, C.POINTER(C.c_int32)]
    lib.stg_argmax_rows.argtypes = [vp, vp, i32, i32, i32, i64, vp, vp]
    lib.stg_argmax_rows_static.argtypes = [vp, i32, i32, i32, i64, vp, vp]
    lib.stg_sample_rows.argtypes = [vp, C.POINTER(StgSampleBatch), vp]
    lib.stg_build_distribution.argtypes = [vp, C.POINTER(StgSampleBatch), vp, vp]
    lib.stg_spec_verify.argtypes = [vp, C.POINTER(StgSpecBatch), vp]
    lib.stg_sample_with_distribution.argtypes = [vp, C.POINTER(StgSampleBatch), vp, vp]
    lib.stg_sample_from_probs.argtypes = [vp, vp, i32, i32, i64, vp, vp, vp, C.c_uint32, vp]
    lib.stg_resample_residual.argtypes = [vp, vp, vp, i32, i32, i64, vp, vp, vp, C.c_uint32, vp]
    lib.stg_mtp_accept.argtypes = [vp, vp, i32, i32, i32, i64, vp, f32, vp, vp, vp, vp]
    lib.stg_and_masks.argtypes = [vp, vp, i32, i32, i32, i64, vp, i64, vp, vp]
    lib.stg_mask_cache_put.argtypes = [vp, C.c_uint64, vp, i32, vp]
    lib.stg_mask_cache_contains.argtypes = [vp, C.c_uint64]
    lib.stg_mask_compose.argtypes = [vp, vp, i32, i32, i32, i32, vp, i64, vp, vp]
    lib.stg_history_reset.argtypes = [vp, i32, i32, vp]
    lib.stg_history_load.argtypes = [vp, i32, vp, i32, vp]
    lib.stg_history_append.argtypes = [vp, vp, i32, vp, vp]
    lib.stg_history_length.argtypes = [vp, i32]
    lib.stg_comm_unique_id.argtypes = [vp]
    lib.stg_comm_init.argtypes = [vp, vp, i32, i32]
    lib.stg_comm_destroy.argtypes = [vp]
    lib.stg_shard_select.argtypes = [vp, C.POINTER(StgSampleBatch), i32, i32, vp]
    lib.stg_shard_allgather.argtypes = [vp, vp]
    lib.stg_shard_exchange_bytes.argtypes = [vp, C.POINTER(C.c_uint64)]
    lib.stg_shard_finish.argtypes = [vp, C.POINTER(StgSampleBatch), i32, vp]
    lib.stg_shard_gather_local.argtypes = [vp, C.POINTER(vp), i32, vp]
    for name in EXPORTS:
        fn = getattr(lib, name)
        if name != "stg_last_error":
            fn.restype = C.c_int
    _lib = lib
    return lib
