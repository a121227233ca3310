// Host-side declarations shared by the translation units of the library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/moe_b200_sampler.h"

#define MOE_SLICE_SLOT_RECORDS 1024u
// largest top_k the small-buffer kernel instantiation serves (the 4 * k + 64 records a slice expects above its sampled
// threshold must fit the 2048-record buffer with room for their spread)
#define MOE_SAMPLER_TOPK_SMALL_MAX 448u
// entries of the router's [expert][block] count table (expert_count * blocks of the select kernel never exceeds it)
#define MOE_ROUTER_BLOCK_TABLE_ENTRIES 262144u

namespace moe {

// Device workspace shared by the kernels of one handle.
struct Workspace
{
    // rows the streaming kernel could not finish; consumed (and reset to 0) by
    // the exact kernel of the same call
    uint32_t* exact_count = nullptr;   // [1]
    uint32_t* exact_done = nullptr;    // [1] CTAs of the exact kernel that have finished
    uint32_t* exact_next = nullptr;    // [1] next entry of exact_rows nobody has taken yet
    uint32_t* exact_rows = nullptr;    // [max_rows]
    // per-slot scratch of the exact kernel: (keys, index) pair 0 then pair 1,
    // each array `max_vocab` rounded up to a multiple of 4 entries
    uint32_t* sort_keys = nullptr;     // [slots][4][stride]
    // publication slots of the streaming kernel when a row is cut into slices:
    // one per CTA, MOE_SLICE_SLOT_RECORDS records and a 4-word header each
    uint64_t* slice_records = nullptr; // [slice_slots][MOE_SLICE_SLOT_RECORDS]
    uint32_t* slice_header = nullptr;  // [slice_slots][4]: count, needs-exact flag, max key, pad
    uint32_t* row_arrivals = nullptr;  // [max_rows] slices of the row that have published (self-resetting)
    uint32_t slice_slots = 0;
    uint32_t slots = 0;
    uint32_t max_rows = 0;
    uint32_t max_vocab = 0;
};

struct SampleArgs
{
    const void* logits;
    int dtype;
    uint32_t rows;
    uint32_t vocab;
    size_t row_stride;
    const moe_row_params* params; // device
    uint64_t step_offset;
    const int32_t* stop_offsets; // device or null
    const int32_t* stop_tokens;  // device or null
    int32_t* token_id;
    float* probability;
    uint32_t* row_flags;   // may be null
    int32_t* row_status;   // may be null
    int32_t* topk_index;   // may be null
    uint32_t topk_stride;
    // optional: every row's kept candidates with their renormalised probabilities
    // (the vector sampling_distribution returns, session.cpp:76-136)
    int32_t* kept_token;     // [rows x kept_stride] or null
    float* kept_probability; // [rows x kept_stride] or null
    uint32_t* kept_count;    // [rows] or null: candidates kept (may exceed kept_stride; the list is cut there)
    uint32_t kept_stride;
    // vocabulary-sharded local pass: write the slice's Top-K records instead of sampling
    uint64_t* candidates_out; // may be null
    uint32_t candidates_k;
    uint32_t vocab_begin;
    // some row has a Top-K too large for the small record buffer: use the
    // large-buffer instantiation (fewer CTAs per SM)
    bool large_top_k;
    // launched with programmatic stream serialization: the kernel may start
    // while the previous kernel of the stream is still finishing, so it waits
    // for that kernel (griddepcontrol.wait) before its first global write
    bool overlap_previous;
};

cudaError_t launch_sample_rows(const SampleArgs& args, const Workspace& ws, uint32_t splits, cudaStream_t stream);
cudaError_t launch_sample_exact(const SampleArgs& args, const Workspace& ws, cudaStream_t stream);
// token_id / probability / row_flags / row_status arrays -> one 16-byte record per row
cudaError_t launch_pack_sampled_rows(const int32_t* token_id, const float* probability, const uint32_t* row_flags, const int32_t* row_status,
                                     uint32_t rows, moe_sampled_row* packed, cudaStream_t stream);
cudaError_t launch_merge_candidates(const uint64_t* gathered, uint32_t shards, uint32_t rows, uint32_t top_k, const moe_row_params* params,
                                    uint64_t step_offset, int32_t* token_id, float* probability, uint32_t* row_flags, int32_t* row_status,
                                    int32_t* topk_index, uint32_t topk_stride, cudaStream_t stream);

// Speculative verification of `sessions` Sessions with draft_count proposals each.  Rows of the row
// outputs and kept lists: Session b's target positions are rows b*(draft_count+1) .. +draft_count,
// its draft positions rows sessions*(draft_count+1) + b*draft_count .. +draft_count-1.
struct SpeculativeArgs
{
    uint32_t sessions;
    uint32_t draft_count;
    uint32_t vocab;
    const moe_row_params* params; // device, by row; a Session's options and counters are those of its first target row
    const int32_t* proposed;      // device, [sessions * draft_count]
    const int32_t* token;         // per-row sampler outputs
    const float* probability;
    const uint32_t* row_flags;
    const int32_t* row_status;
    const int32_t* kept_token;
    const float* kept_probability;
    const uint32_t* kept_count;
    uint32_t kept_stride;
    float* dense;             // [sessions * vocab] scratch: the residual by token id
    int32_t* residual_token;  // [sessions * vocab] scratch: its positive entries in token-id order
    float* residual_value;
    float* accepted_probability; // [sessions * draft_count]
    moe_speculative_result* result; // [sessions]
};

cudaError_t launch_speculative_verify(const SpeculativeArgs& args, cudaStream_t stream);

struct RouterArgs
{
    const float* logits;
    uint32_t token_count;
    moe_router_options options; // pointers are device pointers
    uint32_t* expert_offsets;
    uint32_t* route_token;
    uint32_t* route_rank;
    float* route_weight;
    int32_t* plan_status;
    // scratch
    uint32_t* selected_expert; // [token_count * top_k]
    float* selected_weight;    // [token_count * top_k]
    uint32_t* block_counts;    // [MOE_ROUTER_BLOCK_TABLE_ENTRIES]: routes per (expert, block of the select kernel)
    uint32_t tokens_per_block; // filled in by the launcher
};
struct RouterPartition
{
    uint32_t tokens_per_block;
    uint32_t blocks;
};
// blocks of the select kernel: about four per SM (148 SMs, four warps of one token each per block), fewer when
// the [expert][block] table would outgrow MOE_ROUTER_BLOCK_TABLE_ENTRIES
inline RouterPartition router_partition_host(uint32_t token_count, uint32_t experts)
{
    constexpr uint32_t kWarpsPerBlock = 4;
    RouterPartition part;
    part.tokens_per_block = kWarpsPerBlock * ((token_count + kWarpsPerBlock * 592u - 1u) / (kWarpsPerBlock * 592u));
    if (part.tokens_per_block == 0)
        part.tokens_per_block = kWarpsPerBlock;
    part.blocks = (token_count + part.tokens_per_block - 1u) / part.tokens_per_block;
    while (static_cast<uint64_t>(part.blocks) * experts > MOE_ROUTER_BLOCK_TABLE_ENTRIES)
    {
        part.tokens_per_block *= 2u;
        part.blocks = (token_count + part.tokens_per_block - 1u) / part.tokens_per_block;
    }
    if (part.blocks == 0)
        part.blocks = 1;
    return part;
}
// expert_counts: [expert_count] scratch; scan_done: one word that is 0 between calls; error_word: ~0 between calls
cudaError_t launch_router_dispatch_kernels(const RouterArgs& args, uint32_t* expert_counts, uint32_t* scan_done, unsigned long long* error_word,
                                           cudaStream_t stream);
// out_of_range: one device word, set to 1 when a route_token entry is >= token_count (its row is zero-filled)
cudaError_t launch_regroup_gather(const float* hidden, uint32_t token_count, uint32_t columns, const uint32_t* route_token, uint32_t route_count,
                                  float* gathered, int32_t* out_of_range, cudaStream_t stream);

// Kernels that need more than 48 KiB of dynamic shared memory must opt in with
// cudaFuncSetAttribute, which applies to the current device only: what has been
// configured is remembered per device ordinal (one SharedOptIn per kernel).
constexpr int kMaxDevices = 64;
struct SharedOptIn
{
    size_t bytes[kMaxDevices] = {};
};
// true when `shared_bytes` still has to be configured on `device`; records it as configured
inline bool opt_in_needed(SharedOptIn& state, int device, size_t shared_bytes)
{
    if (device < 0 || device >= kMaxDevices)
        return true; // untracked ordinal: configure on every launch
    if (state.bytes[device] >= shared_bytes)
        return false;
    state.bytes[device] = shared_bytes; // racing host threads write the same value
    return true;
}
template<typename Kernel>
cudaError_t opt_in_shared(SharedOptIn& state, Kernel kernel, size_t shared_bytes)
{
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess)
        return status;
    if (!opt_in_needed(state, device, shared_bytes))
        return cudaSuccess;
    status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared_bytes));
    if (status != cudaSuccess && device >= 0 && device < kMaxDevices)
        state.bytes[device] = 0;
    return status;
}

// Stable Top-K of every row of `scores` (score descending, index ascending): out_index [rows x top_k] in that
// order, 0xFFFFFFFF beyond min(top_k, count); out_score may be null.  top_k <= MOE_INDEXER_TOPK_MAX.
cudaError_t launch_indexer_topk(const float* scores, uint32_t rows, uint32_t count, size_t row_stride, uint32_t top_k, uint32_t* out_index,
                                float* out_score, cudaStream_t stream);

uint32_t choose_splits(uint32_t rows, uint32_t vocab, int dtype, int sm_count, uint32_t slice_slots, bool large_top_k, bool overlapped);

} // namespace moe
