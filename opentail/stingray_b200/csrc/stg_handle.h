// Internal: the handle behind StgHandle and helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../../include/stingray_sampler.h"
#include "stg_launch.h"
#include "stg_types.h"

namespace stg {

struct DevBuf {
    void *p = nullptr;
    size_t bytes = 0;
    bool guarded = false;  // checked build of the handle: kGuardBytes of a fixed pattern follow the buffer
};
constexpr size_t kGuardBytes = 256;
constexpr int kGuardByte = 0xC5;

// The host plan of one sampling step (built by make_plan in stg_api.cu).
struct Plan {
    std::vector<RowPlan> rows;
    std::vector<WorkItem> items;
    std::vector<float> pow_tab;
    int chunk_len = 0;
    int cap = kSubTile + 1;
    bool any_row_item = false;
    int n_row_items = 0;
    size_t smem = 0;
    uint64_t n_greedy = 0, n_topk = 0, n_full = 0;
    int max_topk_path_k = 0;  // largest top_k among the rows on the top-k path
    int max_sel = 1;          // largest selection count of a chunked row
    bool flat = false;        // the chunked rows run as the flat step (stg_flat.cuh)
    bool flat_full = false;   // ... and so do the full-vocabulary rows
    int n_chunk_rows = 0;
    int n_full_without_top_p = 0;  // sampled full-vocabulary rows with top-p off
    int n_full_with_top_p = 0;     // ... and on
};

}  // namespace stg

struct StgSampler_ {
    StgConfig cfg{};
    int sm_count = 0;
    size_t smem_optin = 0;
    std::string err;
    StgStats stats{};
    bool checked = false;                // STG_CHECKED=1 at creation: guard words behind every device buffer
    // replayable steps: the launches of a step whose plan and arguments have been seen before are
    // captured once into a CUDA graph and replayed (stg_api.cu)
    struct StepGraph {
        std::vector<unsigned char> key;
        cudaGraphExec_t exec = nullptr;
        uint64_t used = 0;
        int launches = 0;  // kernels in the graph
    };
    std::vector<StepGraph> graphs;
    std::vector<uint64_t> seen_keys;       // hashes of the last few argument sets that were launched directly
    uint64_t graph_tick = 0;
    uint64_t plan_version = 0;             // bumped with every new plan
    bool graphs_off = false;               // STG_NO_GRAPH=1, or a capture failed on this handle
    int lookback_drill = 0;              // STG_LOOKBACK_DRILL=1 or 2 at creation: see SampleArgs::lookback_drill

    // workspace (allocated once at creation)
    stg::DevBuf plan_dev;                // RowPlan[], WorkItem[], pow table
    unsigned char *plan_host = nullptr;  // pinned mirror ring
    cudaEvent_t plan_ev[4]{};
    int plan_slot = 0;
    std::vector<unsigned char> plan_cache;  // bytes of the plan last uploaded
    stg::Plan plan;                          // the plan of the last step ...
    std::vector<unsigned char> plan_key, plan_key_scratch;  // ... and the batch description it was built for
    bool plan_valid = false;
    const stg::RowPlan *d_rows = nullptr;    // where that plan lives on the device
    const stg::WorkItem *d_items = nullptr;
    const float *d_pow = nullptr;
    stg::DevBuf flat_rows;               // FlatRow per row (stg_flat.cuh)
    // full-vocabulary rows of the flat step: FullWs arrays for up to full_cap rows
    stg::DevBuf fw_rows, fw_e, fw_ov_id, fw_ov_adj, fw_ew, fw_hist, fw_bstart, fw_binexp, fw_flagbits, fw_cursor, fw_keys;
    int full_cap = 0;
    stg::DevBuf cand, cand_count, tickets, work_counter, escratch, keyscratch, listscratch, dists;
    stg::DevBuf st_hist, st_bias_ids, st_bias_vals, st_uniforms, st_mask, st_logits;
    stg::DevBuf o_tokens, o_probs, o_flags, o_topk_ids, o_topk_vals, o_topk_probs, o_pairs;
    stg::DevBuf ticks;                   // diagnostic phase stamps (STG_PHASE_TICKS=1)
    stg::KernelTimer kt;                 // diagnostic events between kernels (STG_KERNEL_TIMES=1)
    int ticks_items = 0;
    stg::DevBuf sp_draft, sp_uniforms, sp_accepted, sp_correction, sp_aprobs, sp_flags, sp_rowstats;
    int64_t escratch_stride = 0, key_stride = 0;
    size_t cand_entries = 0;
    uint32_t work_base = 0, work_base_rows = 0;
    cudaStream_t aux_stream = nullptr;   // lowest priority: the chunked rows' finish runs here, beside the full rows' phases
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_cut = nullptr, ev_exp = nullptr, ev_scatter = nullptr;
    cudaStream_t plan_stream = nullptr;  // the plan and scatter kernels of the full rows, beside the walk
    cudaEvent_t ev_order = nullptr;      // orders a call behind the previous call's work when the stream changes
    cudaStream_t last_stream = nullptr;
    bool last_stream_valid = false;
    size_t plan_bytes_cap = 0;
    // exchange buffers of the vocabulary-sharded mode
    stg::DevBuf xchg_local, xchg_gather;  // per rank: [rows, stride] keys then [rows] counts
    void *nccl_lib = nullptr;
    void *nccl_comm = nullptr;
    int rank = 0, n_ranks = 1;
    int shard_sel = 0, shard_rows = 0, shard_rows_used = 0, shard_stride_used = 0;
    size_t shard_block_bytes = 0;         // bytes one rank contributes to the exchange of the current step
    // device-resident histories (stg_history.cu): slot r at ring_ids + r * max(max_history, 1)
    stg::DevBuf ring_ids, ring_len_dev;
    std::vector<int32_t> ring_len;        // host mirror of the lengths
    std::vector<uint8_t> ring_dropped;    // the slot has dropped its oldest token at least once
    // bitmask cache (stg_mask.cu)
    stg::DevBuf mc_words, mc_slots;       // [max_cached_masks, mc_stride] words; slot indices of one composition
    int64_t mc_stride = 0;
    std::vector<uint64_t> mc_key, mc_used;  // per entry: key (0 = free) and the tick of its last use
    uint64_t mc_tick = 0;
    std::unordered_map<uint64_t, int> mc_index;  // key -> entry
    std::vector<int32_t> mc_slot_scratch;
};

namespace stg {

int fail(StgHandle h, int code, const std::string &msg);
int cuda_fail(StgHandle h, cudaError_t e, const char *what);
int dev_alloc(StgHandle h, DevBuf &b, size_t bytes);
void dev_free(DevBuf &b);
inline size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }
// What distinguishes the callers of the shared batch runner.
struct BatchExtra {
    int mode = 0;                 // 0 sample, 1 materialise distributions, 2 descriptors only
    float *dist_out = nullptr;    // mode 1
    void *pairs_out = nullptr;    // stg_argmax_rows
    RowDist *dists_out = nullptr; // mode 2
    int shard_mode = 0;           // 1: export each row's local candidates to the exchange buffer
    int vocab_offset = 0;
    int global_vocab = 0;         // 0: same as the batch's vocab
};
int run_batch(StgHandle h, const StgSampleBatch *b, const BatchExtra &x, void *stream);
int stage_in(StgHandle h, const void *src, size_t bytes, bool on_host, DevBuf &stage, cudaStream_t stream,
             const void **out);

#define CK(call)                                                        \
    do {                                                                \
        cudaError_t e_ = (call);                                        \
        if (e_ != cudaSuccess) return stg::cuda_fail(h, e_, #call);     \
    } while (0)

}  // namespace stg
