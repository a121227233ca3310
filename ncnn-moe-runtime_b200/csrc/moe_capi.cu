// C ABI of the library (include/moe_b200_sampler.h): handle management,
// argument checks, parameter upload, kernel launches, host-buffer variants.

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "moe_common.cuh"
#include "moe_internal.h"

using namespace moe;

struct moe_sampler
{
    int device = 0;
    int sm_count = 0;
    uint32_t max_rows = 0;
    uint32_t max_vocab = 0;
    Workspace ws;
    cudaStream_t stream = nullptr; // used by the host-buffer entry points

    // resident per-row parameters and stop lists
    moe_row_params* params_dev = nullptr;
    int32_t* stop_offsets_dev = nullptr;
    int32_t* stop_tokens_dev = nullptr;
    size_t stop_tokens_capacity = 0;
    uint32_t resident_rows = 0;
    bool resident_needs_exact = false;
    bool resident_large_top_k = false;
    bool overlap_launches = false;
    bool resident_has_stops = false;

    // packed per-row results of moe_sample_tokens
    moe_sampled_row* sampled_dev = nullptr;

    // staging for the host-buffer entry points
    void* logits_dev = nullptr;
    size_t logits_dev_bytes = 0;
    int32_t* token_dev = nullptr;
    float* probability_dev = nullptr;
    uint32_t* flags_dev = nullptr;
    int32_t* status_dev = nullptr;
    int32_t* topk_dev = nullptr;
    size_t topk_dev_entries = 0;

    // speculative verification scratch (allocated on first use)
    int32_t* spec_kept_token = nullptr;
    float* spec_kept_probability = nullptr;
    uint32_t* spec_kept_count = nullptr;
    int32_t* spec_token = nullptr;
    float* spec_probability = nullptr;
    uint32_t* spec_flags = nullptr;
    int32_t* spec_status = nullptr;
    float* spec_dense = nullptr;
    int32_t* spec_residual_token = nullptr;
    float* spec_residual_value = nullptr;
    size_t spec_list_capacity = 0;  // entries of each kept-list array
    size_t spec_row_capacity = 0;   // entries of each per-row array
    size_t spec_dense_capacity = 0; // entries of each residual array

    // router scratch
    uint32_t* selected_expert = nullptr;
    float* selected_weight = nullptr;
    size_t selected_capacity = 0;
    uint32_t* expert_counts = nullptr;
    size_t expert_counts_capacity = 0;
    unsigned long long* router_error = nullptr;
    uint32_t* router_scan_done = nullptr;    // one word, 0 between calls
    uint32_t* router_block_counts = nullptr; // [MOE_ROUTER_BLOCK_TABLE_ENTRIES], allocated by the first router call
    int32_t* gather_status = nullptr;        // one word: set when moe_regroup_gather met a token index out of range
    // router host staging
    float* router_logits_dev = nullptr;
    size_t router_logits_capacity = 0;
    float* router_bias_dev = nullptr;
    uint32_t* router_explicit_dev = nullptr;
    size_t router_bias_capacity = 0;
    size_t router_explicit_capacity = 0;
    uint32_t* router_offsets_dev = nullptr;
    size_t router_offsets_capacity = 0;
    uint32_t* router_token_dev = nullptr;
    uint32_t* router_rank_dev = nullptr;
    float* router_weight_dev = nullptr;
    size_t router_route_capacity = 0;
    int32_t* router_status_dev = nullptr;

    std::string last_error;
};

namespace {

int fail(moe_sampler* sampler, int status, const std::string& text)
{
    if (sampler != nullptr)
        sampler->last_error = text;
    return status;
}

int fail_cuda(moe_sampler* sampler, cudaError_t error, const char* where)
{
    return fail(sampler, MOE_STATUS_CUDA_ERROR, std::string(where) + ": " + cudaGetErrorString(error));
}

#define MOE_CUDA_CHECK(sampler, call)                          \
    do                                                         \
    {                                                          \
        const cudaError_t moe_cuda_status = (call);            \
        if (moe_cuda_status != cudaSuccess)                    \
            return fail_cuda((sampler), moe_cuda_status, #call); \
    } while (0)

template<typename T>
cudaError_t grow(T*& pointer, size_t& capacity, size_t wanted)
{
    if (wanted <= capacity && pointer != nullptr)
        return cudaSuccess;
    if (pointer != nullptr)
    {
        cudaError_t status = cudaFree(pointer);
        if (status != cudaSuccess)
            return status;
        pointer = nullptr;
        capacity = 0;
    }
    const size_t entries = wanted > 0 ? wanted : 1;
    cudaError_t status = cudaMalloc(reinterpret_cast<void**>(&pointer), entries * sizeof(T));
    if (status == cudaSuccess)
        capacity = entries;
    return status;
}

struct DeviceGuard
{
    int previous = -1;
    explicit DeviceGuard(int device)
    {
        cudaGetDevice(&previous);
        if (previous != device)
            cudaSetDevice(device);
        else
            previous = -1;
    }
    ~DeviceGuard()
    {
        if (previous >= 0)
            cudaSetDevice(previous);
    }
};

// Uploads per-row parameters (and stop lists) and records what the rows may need.
int upload_rows(moe_sampler* sampler, cudaStream_t stream, uint32_t rows, const moe_row_params* params, const int32_t* stop_offsets,
                const int32_t* stop_tokens)
{
    bool needs_exact = false;
    bool large_top_k = false;
    for (uint32_t row = 0; row < rows; ++row)
    {
        const moe_row_params& p = params[row];
        if (validate_row(p) != MOE_ROW_OK || p.temperature == 0.0f)
            continue;
        if (p.top_k == 0 || p.top_k > MOE_SAMPLER_TOPK_FAST_MAX)
            needs_exact = true;
        else if (p.top_k > MOE_SAMPLER_TOPK_SMALL_MAX)
            large_top_k = true;
    }
    // pageable source: the runtime stages the bytes before returning, so the
    // caller's array may be reused at once
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(sampler->params_dev, params, sizeof(moe_row_params) * rows, cudaMemcpyHostToDevice, stream));
    sampler->resident_has_stops = false;
    if (stop_offsets != nullptr && stop_tokens != nullptr)
    {
        const size_t total = static_cast<size_t>(stop_offsets[rows]);
        if (total > 0)
        {
            if (total > sampler->stop_tokens_capacity)
            {
                MOE_CUDA_CHECK(sampler, cudaStreamSynchronize(stream));
                MOE_CUDA_CHECK(sampler, grow(sampler->stop_tokens_dev, sampler->stop_tokens_capacity, total));
            }
            MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(sampler->stop_offsets_dev, stop_offsets, sizeof(int32_t) * (rows + 1), cudaMemcpyHostToDevice, stream));
            MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(sampler->stop_tokens_dev, stop_tokens, sizeof(int32_t) * total, cudaMemcpyHostToDevice, stream));
            sampler->resident_has_stops = true;
        }
    }
    sampler->resident_rows = rows;
    sampler->resident_needs_exact = needs_exact;
    sampler->resident_large_top_k = large_top_k;
    return MOE_STATUS_OK;
}

// The exact kernel's per-slot sort scratch (16 bytes per vocabulary entry and
// slot) is only needed by batches that contain rows without Top-K: it is
// allocated when the first such batch arrives, not with the handle.
int ensure_exact_scratch(moe_sampler* sampler, cudaStream_t stream)
{
    Workspace& ws = sampler->ws;
    if (ws.sort_keys != nullptr)
        return MOE_STATUS_OK;
    const size_t stride = (static_cast<size_t>(ws.max_vocab) + 3u) & ~static_cast<size_t>(3u);
    MOE_CUDA_CHECK(sampler, cudaStreamSynchronize(stream));
    MOE_CUDA_CHECK(sampler, cudaMalloc(reinterpret_cast<void**>(&ws.sort_keys), sizeof(uint32_t) * 4u * stride * ws.slots));
    return MOE_STATUS_OK;
}

// Slices per row; MOE_B200_SPLITS (1..32) overrides the built-in policy for tuning runs.
uint32_t pick_splits(const moe_sampler* sampler, uint32_t rows, uint32_t vocab, int dtype, bool large_top_k, bool overlapped = false)
{
    uint32_t splits = choose_splits(rows, vocab, dtype, sampler->sm_count, sampler->ws.slice_slots, large_top_k, overlapped);
    if (const char* forced = std::getenv("MOE_B200_SPLITS"))
    {
        const long value = std::strtol(forced, nullptr, 10);
        if (value >= 1 && value <= 32 && static_cast<uint64_t>(rows) * value <= sampler->ws.slice_slots)
            splits = static_cast<uint32_t>(value);
    }
    return splits;
}

int check_shape(moe_sampler* sampler, int dtype, uint32_t rows, uint32_t vocab, size_t row_stride)
{
    if (sampler == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    if (dtype != MOE_DTYPE_F32 && dtype != MOE_DTYPE_BF16)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "dtype must be MOE_DTYPE_F32 or MOE_DTYPE_BF16");
    if (vocab == 0)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "cannot sample empty logits");
    if (rows > sampler->max_rows)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "rows exceed the max_rows the sampler was created with");
    if (vocab > sampler->max_vocab)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "vocab exceeds the max_vocab the sampler was created with");
    if (row_stride < vocab)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "row_stride is smaller than vocab");
    if (vocab > 0x7FFFFFFFu)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "vocab does not fit a 32-bit token id");
    return MOE_STATUS_OK;
}

} // namespace

extern "C" {

int moe_sampler_create(int device, uint32_t max_rows, uint32_t max_vocab, moe_sampler** out)
{
    if (out == nullptr || max_rows == 0 || max_vocab == 0)
        return MOE_STATUS_INVALID_ARGUMENT;
    *out = nullptr;
    int device_count = 0;
    if (cudaGetDeviceCount(&device_count) != cudaSuccess || device < 0 || device >= device_count)
        return MOE_STATUS_CUDA_ERROR;
    cudaDeviceProp properties;
    if (cudaGetDeviceProperties(&properties, device) != cudaSuccess)
        return MOE_STATUS_CUDA_ERROR;
    if (properties.major != 10)
        return MOE_STATUS_CUDA_ERROR; // the kernels are built for sm_100a only
    moe_sampler* sampler = new (std::nothrow) moe_sampler();
    if (sampler == nullptr)
        return MOE_STATUS_INTERNAL_ERROR;
    sampler->device = device;
    sampler->sm_count = properties.multiProcessorCount;
    sampler->max_rows = max_rows;
    sampler->max_vocab = max_vocab;
    DeviceGuard guard(device);
    Workspace& ws = sampler->ws;
    ws.max_rows = max_rows;
    ws.max_vocab = max_vocab;
    ws.slots = max_rows < static_cast<uint32_t>(sampler->sm_count) ? max_rows : static_cast<uint32_t>(sampler->sm_count);
    cudaError_t status = cudaSuccess;
    auto allocate = [&](void** pointer, size_t bytes) {
        if (status == cudaSuccess)
            status = cudaMalloc(pointer, bytes);
    };
    uint32_t* counters = nullptr;
    allocate(reinterpret_cast<void**>(&counters), 3 * sizeof(uint32_t));
    allocate(reinterpret_cast<void**>(&ws.exact_rows), sizeof(uint32_t) * max_rows);
    ws.slice_slots = static_cast<uint32_t>(sampler->sm_count) * 6u * 2u + 64u;
    allocate(reinterpret_cast<void**>(&ws.slice_records), sizeof(uint64_t) * MOE_SLICE_SLOT_RECORDS * ws.slice_slots);
    allocate(reinterpret_cast<void**>(&ws.slice_header), sizeof(uint32_t) * 4u * ws.slice_slots);
    allocate(reinterpret_cast<void**>(&ws.row_arrivals), sizeof(uint32_t) * max_rows);
    allocate(reinterpret_cast<void**>(&sampler->params_dev), sizeof(moe_row_params) * max_rows);
    allocate(reinterpret_cast<void**>(&sampler->stop_offsets_dev), sizeof(int32_t) * (static_cast<size_t>(max_rows) + 1));
    allocate(reinterpret_cast<void**>(&sampler->token_dev), sizeof(int32_t) * max_rows);
    allocate(reinterpret_cast<void**>(&sampler->probability_dev), sizeof(float) * max_rows);
    allocate(reinterpret_cast<void**>(&sampler->flags_dev), sizeof(uint32_t) * max_rows);
    allocate(reinterpret_cast<void**>(&sampler->status_dev), sizeof(int32_t) * max_rows);
    allocate(reinterpret_cast<void**>(&sampler->sampled_dev), sizeof(moe_sampled_row) * max_rows);
    allocate(reinterpret_cast<void**>(&sampler->router_error), sizeof(unsigned long long));
    allocate(reinterpret_cast<void**>(&sampler->router_scan_done), sizeof(uint32_t));
    allocate(reinterpret_cast<void**>(&sampler->gather_status), sizeof(int32_t));
    allocate(reinterpret_cast<void**>(&sampler->router_status_dev), sizeof(int32_t));
    if (status == cudaSuccess)
        status = cudaMemset(counters, 0, 3 * sizeof(uint32_t));
    if (status == cudaSuccess)
        status = cudaMemset(ws.row_arrivals, 0, sizeof(uint32_t) * max_rows);
    if (status == cudaSuccess)
        status = cudaMemset(sampler->router_error, 0xFF, sizeof(unsigned long long));
    if (status == cudaSuccess)
        status = cudaMemset(sampler->router_scan_done, 0, sizeof(uint32_t));
    if (status == cudaSuccess)
        status = cudaMemset(sampler->gather_status, 0, sizeof(int32_t));
    if (status == cudaSuccess)
        status = cudaStreamCreateWithFlags(&sampler->stream, cudaStreamNonBlocking);
    if (status == cudaSuccess)
        status = cudaDeviceSynchronize();
    ws.exact_count = counters;
    ws.exact_done = counters != nullptr ? counters + 1 : nullptr;
    ws.exact_next = counters != nullptr ? counters + 2 : nullptr;
    if (status != cudaSuccess)
    {
        moe_sampler_destroy(sampler);
        return MOE_STATUS_CUDA_ERROR;
    }
    *out = sampler;
    return MOE_STATUS_OK;
}

void moe_sampler_destroy(moe_sampler* sampler)
{
    if (sampler == nullptr)
        return;
    DeviceGuard guard(sampler->device);
    cudaDeviceSynchronize();
    void* pointers[] = {sampler->ws.exact_count, sampler->ws.exact_rows, sampler->ws.sort_keys, sampler->ws.slice_records,
                        sampler->ws.slice_header, sampler->ws.row_arrivals, sampler->params_dev, sampler->stop_offsets_dev,
                        sampler->stop_tokens_dev, sampler->logits_dev, sampler->token_dev, sampler->probability_dev, sampler->flags_dev,
                        sampler->status_dev, sampler->topk_dev, sampler->selected_expert, sampler->selected_weight, sampler->expert_counts,
                        sampler->sampled_dev, sampler->router_error, sampler->router_scan_done, sampler->router_block_counts, sampler->gather_status,
                        sampler->router_logits_dev, sampler->router_bias_dev, sampler->router_explicit_dev,
                        sampler->router_offsets_dev, sampler->router_token_dev, sampler->router_rank_dev, sampler->router_weight_dev,
                        sampler->router_status_dev, sampler->spec_kept_token, sampler->spec_kept_probability, sampler->spec_kept_count,
                        sampler->spec_token, sampler->spec_probability, sampler->spec_flags, sampler->spec_status, sampler->spec_dense,
                        sampler->spec_residual_token, sampler->spec_residual_value};
    for (void* pointer : pointers)
        if (pointer != nullptr)
            cudaFree(pointer);
    if (sampler->stream != nullptr)
        cudaStreamDestroy(sampler->stream);
    delete sampler;
}

int moe_sampler_set_overlap(moe_sampler* sampler, int enable)
{
    if (sampler == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    sampler->overlap_launches = enable != 0;
    return MOE_STATUS_OK;
}

const char* moe_sampler_last_error(const moe_sampler* sampler)
{
    return sampler != nullptr ? sampler->last_error.c_str() : "null sampler handle";
}

const char* moe_row_status_message(int row_status)
{
    switch (row_status)
    {
    case MOE_ROW_OK: return "";
    case MOE_ROW_EMPTY_LOGITS: return "cannot sample empty logits";
    case MOE_ROW_BAD_TEMPERATURE: return "temperature must be finite and non-negative";
    case MOE_ROW_BAD_TOP_P: return "top_p must be in the range (0, 1]";
    case MOE_ROW_BAD_MIN_P: return "min_p must be in the range [0, 1]";
    case MOE_ROW_NO_FINITE_LOGIT: return "sampling requires at least one finite logit";
    case MOE_ROW_INVALID_DISTRIBUTION: return "sampling distribution is invalid";
    case MOE_ROW_WORKSPACE_EXHAUSTED: return "row does not fit the sampler workspace";
    case MOE_ROW_DRAFT_ZERO_PROBABILITY: return "sampled draft token has zero probability";
    case MOE_ROW_RESIDUAL_EMPTY: return "speculative residual distribution is empty";
    default: return "unknown row status";
    }
}

int moe_row_status_error_code(int row_status)
{
    if (row_status == MOE_ROW_OK)
        return MOE_STATUS_OK;
    if (row_status == MOE_ROW_WORKSPACE_EXHAUSTED || row_status == MOE_ROW_DRAFT_ZERO_PROBABILITY || row_status == MOE_ROW_RESIDUAL_EMPTY)
        return MOE_STATUS_INTERNAL_ERROR;
    return MOE_STATUS_INVALID_ARGUMENT;
}

float moe_philox_uniform(uint64_t seed, uint64_t row_id, uint64_t step)
{
    return philox_uniform(seed, row_id, step);
}

int moe_host_alloc(size_t bytes, void** out)
{
    if (out == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    return cudaMallocHost(out, bytes > 0 ? bytes : 1) == cudaSuccess ? MOE_STATUS_OK : MOE_STATUS_CUDA_ERROR;
}

void moe_host_free(void* pointer)
{
    if (pointer != nullptr)
        cudaFreeHost(pointer);
}

int moe_sample_batch(moe_sampler* sampler, void* stream_handle, const void* logits, int dtype, uint32_t rows, uint32_t vocab, size_t row_stride,
                     const moe_row_params* params, uint64_t step_offset, const int32_t* stop_offsets, const int32_t* stop_tokens,
                     int32_t* token_id, float* probability, uint32_t* row_flags, int32_t* row_status, int32_t* topk_index, uint32_t topk_stride)
{
    moe_sample_outputs outputs = {};
    outputs.token_id = token_id;
    outputs.probability = probability;
    outputs.row_flags = row_flags;
    outputs.row_status = row_status;
    outputs.topk_index = topk_index;
    outputs.topk_stride = topk_stride;
    return moe_sample_batch_ex(sampler, stream_handle, logits, dtype, rows, vocab, row_stride, params, step_offset, stop_offsets, stop_tokens, &outputs);
}

int moe_sample_batch_ex(moe_sampler* sampler, void* stream_handle, const void* logits, int dtype, uint32_t rows, uint32_t vocab, size_t row_stride,
                        const moe_row_params* params, uint64_t step_offset, const int32_t* stop_offsets, const int32_t* stop_tokens,
                        const moe_sample_outputs* outputs)
{
    if (int status = check_shape(sampler, dtype, rows, vocab, row_stride))
        return status;
    if (rows == 0)
        return MOE_STATUS_OK;
    if (outputs == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "outputs must not be null");
    int32_t* const token_id = outputs->token_id;
    float* const probability = outputs->probability;
    uint32_t* const row_flags = outputs->row_flags;
    int32_t* const row_status = outputs->row_status;
    int32_t* const topk_index = outputs->topk_index;
    const uint32_t topk_stride = outputs->topk_stride;
    if (logits == nullptr || token_id == nullptr || probability == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "logits, token_id and probability must not be null");
    if (outputs->kept_count == nullptr && (outputs->kept_token != nullptr || outputs->kept_probability != nullptr))
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "kept_token / kept_probability need kept_count");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    DeviceGuard guard(sampler->device);
    if (params != nullptr)
    {
        if (int status = upload_rows(sampler, stream, rows, params, stop_offsets, stop_tokens))
            return status;
    }
    else if (sampler->resident_rows != rows)
    {
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "params is null but no parameters for this row count are resident");
    }
    SampleArgs args = {};
    args.logits = logits;
    args.dtype = dtype;
    args.rows = rows;
    args.vocab = vocab;
    args.row_stride = row_stride;
    args.params = sampler->params_dev;
    args.step_offset = step_offset;
    args.stop_offsets = sampler->resident_has_stops ? sampler->stop_offsets_dev : nullptr;
    args.stop_tokens = sampler->resident_has_stops ? sampler->stop_tokens_dev : nullptr;
    args.token_id = token_id;
    args.probability = probability;
    args.row_flags = row_flags;
    args.row_status = row_status;
    args.topk_index = topk_index;
    args.topk_stride = topk_index != nullptr ? topk_stride : 0;
    args.kept_token = outputs->kept_token;
    args.kept_probability = outputs->kept_probability;
    args.kept_count = outputs->kept_count;
    args.kept_stride = outputs->kept_count != nullptr ? outputs->kept_stride : 0;
    args.large_top_k = sampler->resident_large_top_k;
    args.overlap_previous = sampler->overlap_launches;
    const uint32_t splits = pick_splits(sampler, rows, vocab, dtype, args.large_top_k, args.overlap_previous);
    MOE_CUDA_CHECK(sampler, launch_sample_rows(args, sampler->ws, splits, stream));
    if (sampler->resident_needs_exact)
    {
        if (int status = ensure_exact_scratch(sampler, stream))
            return status;
        MOE_CUDA_CHECK(sampler, launch_sample_exact(args, sampler->ws, stream));
    }
    return MOE_STATUS_OK;
}

int moe_speculative_verify_batch(moe_sampler* sampler, void* stream_handle, const void* target_logits, const void* draft_logits, int dtype,
                                 uint32_t sessions, uint32_t draft_count, uint32_t vocab, size_t row_stride, const int32_t* proposed_tokens,
                                 const moe_row_params* params, float* accepted_probability, moe_speculative_result* results)
{
    if (sampler == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    if (draft_count > MOE_SPECULATIVE_MAX_DRAFT)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "draft_count exceeds MOE_SPECULATIVE_MAX_DRAFT");
    const uint64_t total_rows = static_cast<uint64_t>(sessions) * (2u * draft_count + 1u);
    if (total_rows > sampler->max_rows)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "sessions * (2 * draft_count + 1) exceeds the handle's max_rows");
    if (int status = check_shape(sampler, dtype, static_cast<uint32_t>(total_rows), vocab, row_stride))
        return status;
    if (sessions == 0)
        return MOE_STATUS_OK;
    if (target_logits == nullptr || params == nullptr || results == nullptr ||
        (draft_count > 0 && (draft_logits == nullptr || proposed_tokens == nullptr || accepted_probability == nullptr)))
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "target_logits, draft_logits, proposed_tokens, params, accepted_probability and results must not be null");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    DeviceGuard guard(sampler->device);
    const uint32_t target_rows = sessions * (draft_count + 1u);
    const uint32_t draft_rows = sessions * draft_count;
    const uint32_t rows = target_rows + draft_rows;

    // a kept list is as long as its Session's top_k, or the vocabulary without Top-K
    uint32_t kept_stride = 1;
    for (uint32_t b = 0; b < sessions; ++b)
    {
        const uint32_t k = params[b].top_k;
        kept_stride = std::max(kept_stride, k == 0 || k > vocab ? vocab : k);
    }
    kept_stride = (kept_stride + 3u) & ~3u;
    const size_t list_entries = static_cast<size_t>(rows) * kept_stride;
    const size_t dense_entries = static_cast<size_t>(sessions) * vocab;
    if (list_entries > sampler->spec_list_capacity || rows > sampler->spec_row_capacity || dense_entries > sampler->spec_dense_capacity)
    {
        // work queued on other streams may still read the old buffers
        MOE_CUDA_CHECK(sampler, cudaDeviceSynchronize());
        size_t capacity = sampler->spec_list_capacity;
        MOE_CUDA_CHECK(sampler, grow(sampler->spec_kept_token, capacity, list_entries));
        capacity = sampler->spec_list_capacity;
        MOE_CUDA_CHECK(sampler, grow(sampler->spec_kept_probability, capacity, list_entries));
        sampler->spec_list_capacity = capacity;
        const auto grow_rows = [&](auto*& pointer) {
            size_t row_capacity = sampler->spec_row_capacity;
            return grow(pointer, row_capacity, static_cast<size_t>(rows));
        };
        MOE_CUDA_CHECK(sampler, grow_rows(sampler->spec_kept_count));
        MOE_CUDA_CHECK(sampler, grow_rows(sampler->spec_token));
        MOE_CUDA_CHECK(sampler, grow_rows(sampler->spec_probability));
        MOE_CUDA_CHECK(sampler, grow_rows(sampler->spec_flags));
        MOE_CUDA_CHECK(sampler, grow_rows(sampler->spec_status));
        sampler->spec_row_capacity = std::max<size_t>(sampler->spec_row_capacity, rows);
        const auto grow_dense = [&](auto*& pointer) {
            size_t dense_capacity = sampler->spec_dense_capacity;
            return grow(pointer, dense_capacity, dense_entries);
        };
        MOE_CUDA_CHECK(sampler, grow_dense(sampler->spec_dense));
        MOE_CUDA_CHECK(sampler, grow_dense(sampler->spec_residual_token));
        MOE_CUDA_CHECK(sampler, grow_dense(sampler->spec_residual_value));
        sampler->spec_dense_capacity = std::max(sampler->spec_dense_capacity, dense_entries);
    }
    // every position samples under its Session's options: the target rows first, then the draft rows
    std::vector<moe_row_params> row_params(rows);
    for (uint32_t b = 0; b < sessions; ++b)
    {
        std::fill_n(row_params.begin() + static_cast<size_t>(b) * (draft_count + 1u), draft_count + 1u, params[b]);
        std::fill_n(row_params.begin() + target_rows + static_cast<size_t>(b) * draft_count, draft_count, params[b]);
    }
    if (int status = upload_rows(sampler, stream, rows, row_params.data(), nullptr, nullptr))
        return status;

    SampleArgs args = {};
    args.dtype = dtype;
    args.vocab = vocab;
    args.row_stride = row_stride;
    // the one sample that can be used is that of the target row after all proposals,
    // which the Session would draw with its uniform number draft_count of this step
    args.step_offset = draft_count;
    args.large_top_k = sampler->resident_large_top_k;
    for (int side = 0; side < 2; ++side)
    {
        const uint32_t first = side == 0 ? 0u : target_rows;
        args.logits = side == 0 ? target_logits : draft_logits;
        args.rows = side == 0 ? target_rows : draft_rows;
        if (args.rows == 0)
            continue;
        args.params = sampler->params_dev + first;
        args.token_id = sampler->spec_token + first;
        args.probability = sampler->spec_probability + first;
        args.row_flags = sampler->spec_flags + first;
        args.row_status = sampler->spec_status + first;
        args.kept_token = sampler->spec_kept_token + static_cast<size_t>(first) * kept_stride;
        args.kept_probability = sampler->spec_kept_probability + static_cast<size_t>(first) * kept_stride;
        args.kept_count = sampler->spec_kept_count + first;
        args.kept_stride = kept_stride;
        const uint32_t splits = pick_splits(sampler, args.rows, vocab, dtype, args.large_top_k);
        MOE_CUDA_CHECK(sampler, launch_sample_rows(args, sampler->ws, splits, stream));
        if (sampler->resident_needs_exact)
        {
            if (int status = ensure_exact_scratch(sampler, stream))
                return status;
            MOE_CUDA_CHECK(sampler, launch_sample_exact(args, sampler->ws, stream));
        }
    }
    SpeculativeArgs verify = {};
    verify.sessions = sessions;
    verify.draft_count = draft_count;
    verify.vocab = vocab;
    verify.params = sampler->params_dev;
    verify.proposed = proposed_tokens;
    verify.token = sampler->spec_token;
    verify.probability = sampler->spec_probability;
    verify.row_flags = sampler->spec_flags;
    verify.row_status = sampler->spec_status;
    verify.kept_token = sampler->spec_kept_token;
    verify.kept_probability = sampler->spec_kept_probability;
    verify.kept_count = sampler->spec_kept_count;
    verify.kept_stride = kept_stride;
    verify.dense = sampler->spec_dense;
    verify.residual_token = sampler->spec_residual_token;
    verify.residual_value = sampler->spec_residual_value;
    verify.accepted_probability = accepted_probability;
    verify.result = results;
    MOE_CUDA_CHECK(sampler, launch_speculative_verify(verify, stream));
    return MOE_STATUS_OK;
}

int moe_speculative_verify(moe_sampler* sampler, void* stream_handle, const void* target_logits, const void* draft_logits, int dtype,
                           uint32_t draft_count, uint32_t vocab, size_t row_stride, const int32_t* proposed_tokens,
                           const moe_row_params* params, float* accepted_probability, moe_speculative_result* result)
{
    return moe_speculative_verify_batch(sampler, stream_handle, target_logits, draft_logits, dtype, 1, draft_count, vocab, row_stride, proposed_tokens,
                                        params, accepted_probability, result);
}

int moe_sample_batch_host(moe_sampler* sampler, const void* logits, int dtype, uint32_t rows, uint32_t vocab, size_t row_stride,
                          const moe_row_params* params, const int32_t* stop_offsets, const int32_t* stop_tokens, int32_t* token_id,
                          float* probability, uint32_t* row_flags, int32_t* row_status, int32_t* topk_index, uint32_t topk_stride)
{
    if (int status = check_shape(sampler, dtype, rows, vocab, row_stride))
        return status;
    if (rows == 0)
        return MOE_STATUS_OK;
    if (logits == nullptr || params == nullptr || token_id == nullptr || probability == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "logits, params, token_id and probability must not be null");
    DeviceGuard guard(sampler->device);
    cudaStream_t stream = sampler->stream;
    const size_t element = dtype == MOE_DTYPE_F32 ? 4 : 2;
    const size_t bytes = ((static_cast<size_t>(rows) - 1) * row_stride + vocab) * element;
    if (bytes > sampler->logits_dev_bytes)
    {
        unsigned char* pointer = static_cast<unsigned char*>(sampler->logits_dev);
        MOE_CUDA_CHECK(sampler, grow(pointer, sampler->logits_dev_bytes, bytes));
        sampler->logits_dev = pointer;
    }
    const size_t topk_entries = topk_index != nullptr ? static_cast<size_t>(rows) * topk_stride : 0;
    if (topk_entries > sampler->topk_dev_entries)
        MOE_CUDA_CHECK(sampler, grow(sampler->topk_dev, sampler->topk_dev_entries, topk_entries));
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(sampler->logits_dev, logits, bytes, cudaMemcpyHostToDevice, stream));
    const int status = moe_sample_batch(sampler, stream, sampler->logits_dev, dtype, rows, vocab, row_stride, params, 0, stop_offsets, stop_tokens,
                                        sampler->token_dev, sampler->probability_dev, sampler->flags_dev, sampler->status_dev,
                                        topk_entries > 0 ? sampler->topk_dev : nullptr, topk_stride);
    if (status != MOE_STATUS_OK)
        return status;
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(token_id, sampler->token_dev, sizeof(int32_t) * rows, cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(probability, sampler->probability_dev, sizeof(float) * rows, cudaMemcpyDeviceToHost, stream));
    if (row_flags != nullptr)
        MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(row_flags, sampler->flags_dev, sizeof(uint32_t) * rows, cudaMemcpyDeviceToHost, stream));
    if (row_status != nullptr)
        MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(row_status, sampler->status_dev, sizeof(int32_t) * rows, cudaMemcpyDeviceToHost, stream));
    if (topk_entries > 0)
        MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(topk_index, sampler->topk_dev, sizeof(int32_t) * topk_entries, cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaStreamSynchronize(stream));
    return MOE_STATUS_OK;
}

int moe_sample_tokens(moe_sampler* sampler, void* stream_handle, const void* logits, int dtype, uint32_t rows, uint32_t vocab, size_t row_stride,
                      const moe_row_params* params, uint64_t step_offset, const int32_t* stop_offsets, const int32_t* stop_tokens,
                      moe_sampled_row* results)
{
    if (int status = check_shape(sampler, dtype, rows, vocab, row_stride))
        return status;
    if (rows == 0)
        return MOE_STATUS_OK;
    if (logits == nullptr || results == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "logits and results must not be null");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    const int status = moe_sample_batch(sampler, stream, logits, dtype, rows, vocab, row_stride, params, step_offset, stop_offsets, stop_tokens,
                                        sampler->token_dev, sampler->probability_dev, sampler->flags_dev, sampler->status_dev, nullptr, 0);
    if (status != MOE_STATUS_OK)
        return status;
    DeviceGuard guard(sampler->device);
    MOE_CUDA_CHECK(sampler, launch_pack_sampled_rows(sampler->token_dev, sampler->probability_dev, sampler->flags_dev, sampler->status_dev, rows,
                                                     sampler->sampled_dev, stream));
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(results, sampler->sampled_dev, sizeof(moe_sampled_row) * rows, cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaStreamSynchronize(stream));
    return MOE_STATUS_OK;
}

int moe_speculative_verify_host(moe_sampler* sampler, const void* target_logits, const void* draft_logits, int dtype, uint32_t draft_count,
                                uint32_t vocab, size_t row_stride, const int32_t* proposed_tokens, const moe_row_params* params,
                                float* accepted_probability, moe_speculative_result* result)
{
    const uint32_t rows = 2u * draft_count + 1u;
    if (int status = check_shape(sampler, dtype, rows, vocab, row_stride))
        return status;
    if (draft_count > MOE_SPECULATIVE_MAX_DRAFT)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "draft_count exceeds MOE_SPECULATIVE_MAX_DRAFT");
    if (target_logits == nullptr || params == nullptr || result == nullptr ||
        (draft_count > 0 && (draft_logits == nullptr || proposed_tokens == nullptr || accepted_probability == nullptr)))
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "target_logits, draft_logits, proposed_tokens, params, accepted_probability and result must not be null");
    DeviceGuard guard(sampler->device);
    cudaStream_t stream = sampler->stream;
    const size_t element = dtype == MOE_DTYPE_F32 ? 4 : 2;
    const size_t target_bytes = (static_cast<size_t>(draft_count) * row_stride + vocab) * element;
    const size_t draft_bytes = draft_count > 0 ? ((static_cast<size_t>(draft_count) - 1) * row_stride + vocab) * element : 0;
    const size_t draft_offset = (target_bytes + 255u) & ~static_cast<size_t>(255u);
    // staging: both logit blocks, then the proposed tokens, the accepted probabilities and the result record
    const size_t tokens_offset = (draft_offset + draft_bytes + 255u) & ~static_cast<size_t>(255u);
    const size_t accepted_offset = tokens_offset + sizeof(int32_t) * MOE_SPECULATIVE_MAX_DRAFT;
    const size_t result_offset = accepted_offset + sizeof(float) * MOE_SPECULATIVE_MAX_DRAFT;
    const size_t bytes = result_offset + sizeof(moe_speculative_result);
    if (bytes > sampler->logits_dev_bytes)
    {
        unsigned char* pointer = static_cast<unsigned char*>(sampler->logits_dev);
        MOE_CUDA_CHECK(sampler, grow(pointer, sampler->logits_dev_bytes, bytes));
        sampler->logits_dev = pointer;
    }
    unsigned char* const staging = static_cast<unsigned char*>(sampler->logits_dev);
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(staging, target_logits, target_bytes, cudaMemcpyHostToDevice, stream));
    if (draft_count > 0)
    {
        MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(staging + draft_offset, draft_logits, draft_bytes, cudaMemcpyHostToDevice, stream));
        MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(staging + tokens_offset, proposed_tokens, sizeof(int32_t) * draft_count, cudaMemcpyHostToDevice, stream));
    }
    const int status = moe_speculative_verify(sampler, stream, staging, staging + draft_offset, dtype, draft_count, vocab, row_stride,
                                              reinterpret_cast<const int32_t*>(staging + tokens_offset), params,
                                              reinterpret_cast<float*>(staging + accepted_offset),
                                              reinterpret_cast<moe_speculative_result*>(staging + result_offset));
    if (status != MOE_STATUS_OK)
        return status;
    if (draft_count > 0)
        MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(accepted_probability, staging + accepted_offset, sizeof(float) * draft_count, cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(result, staging + result_offset, sizeof(moe_speculative_result), cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaStreamSynchronize(stream));
    return MOE_STATUS_OK;
}

int moe_sample_local_candidates(moe_sampler* sampler, void* stream_handle, const void* logits, int dtype, uint32_t rows, uint32_t vocab,
                                size_t row_stride, uint32_t vocab_begin, uint32_t top_k, uint64_t* candidates)
{
    if (int status = check_shape(sampler, dtype, rows, vocab, row_stride))
        return status;
    if (top_k == 0 || top_k > MOE_SAMPLER_TOPK_FAST_MAX)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "vocabulary-sharded sampling needs 0 < top_k <= MOE_SAMPLER_TOPK_FAST_MAX");
    if (logits == nullptr || candidates == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "logits and candidates must not be null");
    if (rows == 0)
        return MOE_STATUS_OK;
    DeviceGuard guard(sampler->device);
    SampleArgs args = {};
    args.logits = logits;
    args.dtype = dtype;
    args.rows = rows;
    args.vocab = vocab;
    args.row_stride = row_stride;
    args.candidates_out = candidates;
    args.candidates_k = top_k;
    args.vocab_begin = vocab_begin;
    args.large_top_k = top_k > MOE_SAMPLER_TOPK_SMALL_MAX;
    const uint32_t splits = pick_splits(sampler, rows, vocab, dtype, args.large_top_k);
    MOE_CUDA_CHECK(sampler, launch_sample_rows(args, sampler->ws, splits, static_cast<cudaStream_t>(stream_handle)));
    return MOE_STATUS_OK;
}

int moe_sample_merge_candidates(moe_sampler* sampler, void* stream_handle, const uint64_t* gathered, uint32_t shards, uint32_t rows, uint32_t top_k,
                                const moe_row_params* params, uint64_t step_offset, int32_t* token_id, float* probability, uint32_t* row_flags,
                                int32_t* row_status, int32_t* topk_index, uint32_t topk_stride)
{
    if (sampler == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    if (rows > sampler->max_rows)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "rows exceed the max_rows the sampler was created with");
    if (top_k == 0 || top_k > MOE_SAMPLER_TOPK_FAST_MAX || shards == 0)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "vocabulary-sharded sampling needs shards > 0 and 0 < top_k <= MOE_SAMPLER_TOPK_FAST_MAX");
    if (gathered == nullptr || token_id == nullptr || probability == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "gathered, token_id and probability must not be null");
    if (rows == 0)
        return MOE_STATUS_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    DeviceGuard guard(sampler->device);
    if (params != nullptr)
    {
        if (int status = upload_rows(sampler, stream, rows, params, nullptr, nullptr))
            return status;
    }
    else if (sampler->resident_rows != rows)
    {
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "params is null but no parameters for this row count are resident");
    }
    MOE_CUDA_CHECK(sampler, launch_merge_candidates(gathered, shards, rows, top_k, sampler->params_dev, step_offset, token_id, probability, row_flags,
                                                    row_status, topk_index, topk_index != nullptr ? topk_stride : 0, stream));
    return MOE_STATUS_OK;
}

const char* moe_router_status_message(int plan_status)
{
    switch (plan_status)
    {
    case 0: return "";
    case 101: return "router logits must be finite";
    case 102: return "explicit expert id is out of range";
    case 103: return "selected router weights have a non-positive sum";
    case 104: return "expert dispatch requires at least one token";
    case 105: return "expert dispatch requires 0 < top_k <= expert_count";
    case 106: return "router logits shape does not match token and expert counts";
    case 107: return "router selection bias must match expert_count";
    case 108: return "explicit expert ids must match token_count * top_k";
    case 109: return "routed scaling factor must be finite and positive";
    case 110: return "expert_count exceeds the router kernel's limit of 4096";
    default: return "unknown router status";
    }
}

int moe_router_status_error_code(int plan_status)
{
    if (plan_status == 0)
        return MOE_STATUS_OK;
    if (plan_status == 103)
        return MOE_STATUS_INVALID_MODEL;
    if (plan_status == 110)
        return MOE_STATUS_UNSUPPORTED_MODEL;
    return MOE_STATUS_INVALID_ARGUMENT;
}

int moe_router_check_options(uint32_t token_count, const moe_router_options* options)
{
    // the data-independent checks of expert_dispatcher.cpp:81-96, in its order
    if (options == nullptr)
        return 105;
    if (token_count == 0)
        return 104;
    if (options->expert_count == 0 || options->top_k == 0 || options->top_k > options->expert_count)
        return 105;
    const float scaling = options->routed_scaling_factor;
    if (!(scaling - scaling == 0.0f) || scaling <= 0.0f)
        return 109;
    if (options->expert_count > 4096)
        return 110;
    return 0;
}

int moe_router_dispatch(moe_sampler* sampler, void* stream_handle, const float* router_logits, uint32_t token_count,
                        const moe_router_options* options, uint32_t* expert_offsets, uint32_t* route_token, uint32_t* route_rank,
                        float* route_weight, int32_t* plan_status)
{
    if (sampler == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    const int precheck = moe_router_check_options(token_count, options);
    if (precheck != 0)
        return fail(sampler, moe_router_status_error_code(precheck), moe_router_status_message(precheck));
    if (router_logits == nullptr || expert_offsets == nullptr || route_token == nullptr || route_rank == nullptr || route_weight == nullptr ||
        plan_status == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "router buffers must not be null");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    DeviceGuard guard(sampler->device);
    const size_t routes = static_cast<size_t>(token_count) * options->top_k;
    if (routes > sampler->selected_capacity || options->expert_count > sampler->expert_counts_capacity || sampler->router_block_counts == nullptr)
    {
        // earlier calls on this stream may still use the scratch that is replaced here
        MOE_CUDA_CHECK(sampler, cudaStreamSynchronize(stream));
        if (routes > sampler->selected_capacity)
        {
            size_t capacity = sampler->selected_capacity;
            MOE_CUDA_CHECK(sampler, grow(sampler->selected_expert, capacity, routes));
            MOE_CUDA_CHECK(sampler, grow(sampler->selected_weight, sampler->selected_capacity, routes));
        }
        // every call rewrites the counts it reads (per block, then per expert): nothing to clear
        if (options->expert_count > sampler->expert_counts_capacity)
            MOE_CUDA_CHECK(sampler, grow(sampler->expert_counts, sampler->expert_counts_capacity, options->expert_count));
        if (sampler->router_block_counts == nullptr)
        {
            size_t capacity = 0;
            MOE_CUDA_CHECK(sampler, grow(sampler->router_block_counts, capacity, MOE_ROUTER_BLOCK_TABLE_ENTRIES));
        }
    }
    RouterArgs args = {};
    args.logits = router_logits;
    args.token_count = token_count;
    args.options = *options;
    args.expert_offsets = expert_offsets;
    args.route_token = route_token;
    args.route_rank = route_rank;
    args.route_weight = route_weight;
    args.plan_status = plan_status;
    args.selected_expert = sampler->selected_expert;
    args.selected_weight = sampler->selected_weight;
    args.block_counts = sampler->router_block_counts;
    MOE_CUDA_CHECK(sampler, launch_router_dispatch_kernels(args, sampler->expert_counts, sampler->router_scan_done, sampler->router_error, stream));
    return MOE_STATUS_OK;
}

int moe_router_dispatch_host(moe_sampler* sampler, const float* router_logits, uint32_t token_count, const moe_router_options* options,
                             uint32_t* expert_offsets, uint32_t* route_token, uint32_t* route_rank, float* route_weight, int32_t* plan_status)
{
    if (sampler == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    const int precheck = moe_router_check_options(token_count, options);
    if (precheck != 0)
    {
        if (plan_status != nullptr)
            *plan_status = precheck;
        return fail(sampler, moe_router_status_error_code(precheck), moe_router_status_message(precheck));
    }
    if (router_logits == nullptr || expert_offsets == nullptr || route_token == nullptr || route_rank == nullptr || route_weight == nullptr ||
        plan_status == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "router buffers must not be null");
    DeviceGuard guard(sampler->device);
    cudaStream_t stream = sampler->stream;
    const uint32_t experts = options->expert_count;
    const size_t logit_count = static_cast<size_t>(token_count) * experts;
    const size_t routes = static_cast<size_t>(token_count) * options->top_k;
    MOE_CUDA_CHECK(sampler, grow(sampler->router_logits_dev, sampler->router_logits_capacity, logit_count));
    MOE_CUDA_CHECK(sampler, grow(sampler->router_offsets_dev, sampler->router_offsets_capacity, static_cast<size_t>(experts) + 1));
    if (routes > sampler->router_route_capacity)
    {
        size_t a = sampler->router_route_capacity, b = sampler->router_route_capacity;
        MOE_CUDA_CHECK(sampler, grow(sampler->router_token_dev, a, routes));
        MOE_CUDA_CHECK(sampler, grow(sampler->router_rank_dev, b, routes));
        MOE_CUDA_CHECK(sampler, grow(sampler->router_weight_dev, sampler->router_route_capacity, routes));
    }
    moe_router_options device_options = *options;
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(sampler->router_logits_dev, router_logits, sizeof(float) * logit_count, cudaMemcpyHostToDevice, stream));
    if (options->selection_bias != nullptr)
    {
        MOE_CUDA_CHECK(sampler, grow(sampler->router_bias_dev, sampler->router_bias_capacity, experts));
        MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(sampler->router_bias_dev, options->selection_bias, sizeof(float) * experts, cudaMemcpyHostToDevice, stream));
        device_options.selection_bias = sampler->router_bias_dev;
    }
    if (options->explicit_expert_ids != nullptr)
    {
        MOE_CUDA_CHECK(sampler, grow(sampler->router_explicit_dev, sampler->router_explicit_capacity, routes));
        MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(sampler->router_explicit_dev, options->explicit_expert_ids, sizeof(uint32_t) * routes, cudaMemcpyHostToDevice, stream));
        device_options.explicit_expert_ids = sampler->router_explicit_dev;
    }
    const int status = moe_router_dispatch(sampler, stream, sampler->router_logits_dev, token_count, &device_options, sampler->router_offsets_dev,
                                           sampler->router_token_dev, sampler->router_rank_dev, sampler->router_weight_dev, sampler->router_status_dev);
    if (status != MOE_STATUS_OK)
        return status;
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(plan_status, sampler->router_status_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(expert_offsets, sampler->router_offsets_dev, sizeof(uint32_t) * (experts + 1), cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(route_token, sampler->router_token_dev, sizeof(uint32_t) * routes, cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(route_rank, sampler->router_rank_dev, sizeof(uint32_t) * routes, cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(route_weight, sampler->router_weight_dev, sizeof(float) * routes, cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaStreamSynchronize(stream));
    if (*plan_status != 0)
        return fail(sampler, moe_router_status_error_code(*plan_status), moe_router_status_message(*plan_status));
    return MOE_STATUS_OK;
}

int moe_regroup_gather(moe_sampler* sampler, void* stream_handle, const float* hidden, uint32_t token_count, uint32_t columns,
                       const uint32_t* route_token, uint32_t route_count, float* gathered)
{
    if (sampler == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    if (route_count == 0 || columns == 0)
        return MOE_STATUS_OK;
    if (hidden == nullptr || route_token == nullptr || gathered == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "gather buffers must not be null");
    DeviceGuard guard(sampler->device);
    MOE_CUDA_CHECK(sampler, launch_regroup_gather(hidden, token_count, columns, route_token, route_count, gathered, sampler->gather_status,
                                                  static_cast<cudaStream_t>(stream_handle)));
    return MOE_STATUS_OK;
}

int moe_indexer_topk(moe_sampler* sampler, void* stream_handle, const float* scores, uint32_t rows, uint32_t count, size_t row_stride, uint32_t top_k,
                     uint32_t* out_index, float* out_score)
{
    if (sampler == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    if (top_k == 0 || top_k > MOE_INDEXER_TOPK_MAX)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "indexer Top-K needs 0 < top_k <= MOE_INDEXER_TOPK_MAX");
    if (row_stride < count)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "row_stride is smaller than count");
    if (rows == 0)
        return MOE_STATUS_OK;
    if (scores == nullptr || out_index == nullptr)
        return fail(sampler, MOE_STATUS_INVALID_ARGUMENT, "scores and out_index must not be null");
    DeviceGuard guard(sampler->device);
    MOE_CUDA_CHECK(sampler, launch_indexer_topk(scores, rows, count, row_stride, top_k, out_index, out_score, static_cast<cudaStream_t>(stream_handle)));
    return MOE_STATUS_OK;
}

int moe_regroup_gather_check(moe_sampler* sampler, void* stream_handle, int32_t* out_of_range)
{
    if (sampler == nullptr || out_of_range == nullptr)
        return MOE_STATUS_INVALID_ARGUMENT;
    DeviceGuard guard(sampler->device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    MOE_CUDA_CHECK(sampler, cudaMemcpyAsync(out_of_range, sampler->gather_status, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    MOE_CUDA_CHECK(sampler, cudaMemsetAsync(sampler->gather_status, 0, sizeof(int32_t), stream));
    MOE_CUDA_CHECK(sampler, cudaStreamSynchronize(stream));
    return MOE_STATUS_OK;
}

} // extern "C"
