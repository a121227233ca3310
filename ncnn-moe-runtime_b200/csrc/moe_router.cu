// MoE router: scoring, stable Top-K, weights and grouping by expert.
// Replaces ExpertDispatcher::dispatch (src/graph/expert_dispatcher.cpp:79-158)
// and gather_tokens (src/engine/cpu_executor.cpp:635-642).
//
// Kernel 1 (one warp per token): scores in the reference's arithmetic
//   (softmax with an index-order sequential sum, sigmoid, sqrt-softplus;
//   expert_dispatcher.cpp:24-59), selection key = score + bias, k rounds of a
//   warp-wide arg-max on (key descending, expert id ascending) records — the
//   same record/ordering primitive the sampler uses — then the rank-order
//   sequential sum of the unbiased scores and the weights (:131-144).
// Kernel 2 (one CTA): per-expert counts -> CSR offsets, call status.
// Kernel 3 (one CTA per expert): stable compaction of that expert's routes in
//   (token, rank) order, which is the order the reference appends them in.

#include <cstdio>

#include "moe_common.cuh"
#include "moe_internal.h"

namespace moe {

namespace {

constexpr int kRouteThreads = 128;
constexpr int kRouteWarps = kRouteThreads / 32;

// error word: smaller wins.  class 0 = non-finite logits (the reference checks
// all logits before any token, :97-101), class 1 = first failing token.
__device__ __forceinline__ void report_error(unsigned long long* error_word, uint32_t error_class, uint32_t token, uint32_t code)
{
    const unsigned long long value = (static_cast<unsigned long long>(error_class) << 40) | (static_cast<unsigned long long>(token) << 8) | code;
    atomicMin(error_word, value);
}

__device__ __forceinline__ float router_softplus(float x)
{
    if (x > 20.0f)
        return x;
    if (x < -20.0f)
        return exact_expf(x);
    return exact_log1pf(exact_expf(x));
}

__global__ void __launch_bounds__(kRouteThreads) router_select_kernel(const RouterArgs a, uint32_t* expert_counts, unsigned long long* error_word)
{
    extern __shared__ __align__(16) unsigned char shared_raw[];
    const uint32_t experts = a.options.expert_count;
    const uint32_t top_k = a.options.top_k;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float* scores = reinterpret_cast<float*>(shared_raw) + static_cast<size_t>(warp) * experts;
    uint64_t* records = reinterpret_cast<uint64_t*>(shared_raw + sizeof(float) * experts * kRouteWarps) + static_cast<size_t>(warp) * experts;
    const bool renormalize = (a.options.flags & MOE_ROUTER_FLAG_NORMALIZE_TOPK) != 0 || a.options.normalization == 1;

    for (uint32_t token = blockIdx.x * kRouteWarps + warp; token < a.token_count; token += gridDim.x * kRouteWarps)
    {
        const float* logits = a.logits + static_cast<size_t>(token) * experts;
        bool bad = false;
        float peak = -INFINITY;
        for (uint32_t e = lane; e < experts; e += 32)
        {
            const float v = logits[e];
            bad |= !(fabsf(v) < INFINITY);
            peak = fmaxf(peak, v);
        }
        if (__any_sync(kFullMask, bad))
        {
            if (lane == 0)
                report_error(error_word, 0, 0, 101);
            continue;
        }
        if (a.options.score_function == MOE_ROUTER_SOFTMAX)
        {
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1)
                peak = fmaxf(peak, __shfl_xor_sync(kFullMask, peak, offset));
            float total = 0.0f;
            for (uint32_t base = 0; base < experts; base += 32)
            {
                const uint32_t e = base + lane;
                float weight = 0.0f;
                if (e < experts)
                {
                    weight = exact_expf(__fsub_rn(logits[e], peak));
                    scores[e] = weight;
                }
                const uint32_t steps = min(32u, experts - base);
                for (uint32_t j = 0; j < steps; ++j)
                    total = __fadd_rn(total, __shfl_sync(kFullMask, weight, j)); // index order, :47-51
            }
            __syncwarp();
            for (uint32_t e = lane; e < experts; e += 32)
                scores[e] = __fdiv_rn(scores[e], total);
        }
        else
        {
            for (uint32_t e = lane; e < experts; e += 32)
            {
                const float v = logits[e];
                float score;
                if (a.options.score_function == MOE_ROUTER_SIGMOID)
                    score = __fdiv_rn(1.0f, __fadd_rn(1.0f, exact_expf(-v)));
                else
                    score = __fsqrt_rn(router_softplus(v));
                scores[e] = score;
            }
        }
        __syncwarp();

        float chosen_total = 0.0f;
        uint32_t* out_expert = a.selected_expert + static_cast<size_t>(token) * top_k;
        float* out_weight = a.selected_weight + static_cast<size_t>(token) * top_k;
        bool token_failed = false;
        if (a.options.explicit_expert_ids != nullptr)
        {
            const uint32_t* explicit_ids = a.options.explicit_expert_ids + static_cast<size_t>(token) * top_k;
            uint32_t first_bad = 0xFFFFFFFFu;
            for (uint32_t r = lane; r < top_k; r += 32)
            {
                const uint32_t expert = explicit_ids[r];
                if (expert >= experts)
                    first_bad = min(first_bad, r);
                else
                    out_expert[r] = expert;
            }
            if (__any_sync(kFullMask, first_bad != 0xFFFFFFFFu))
            {
                if (lane == 0)
                    report_error(error_word, 1, token, 102);
                token_failed = true;
            }
        }
        else
        {
            for (uint32_t e = lane; e < experts; e += 32)
            {
                const float key = (a.options.selection_bias != nullptr) ? __fadd_rn(scores[e], a.options.selection_bias[e]) : scores[e];
                // NaN keys never win a `>` compare in the reference; rank them last
                records[e] = (key == key) ? make_record(ordered_key(key), e) : 0ull;
            }
            __syncwarp();
            for (uint32_t r = 0; r < top_k; ++r)
            {
                uint64_t best = 0ull;
                for (uint32_t e = lane; e < experts; e += 32)
                    best = (records[e] > best) ? records[e] : best;
                const uint32_t best_hi = __reduce_max_sync(kFullMask, static_cast<uint32_t>(best >> 32));
                const uint32_t candidate_lo = (static_cast<uint32_t>(best >> 32) == best_hi) ? static_cast<uint32_t>(best) : 0u;
                const uint32_t best_lo = __reduce_max_sync(kFullMask, candidate_lo);
                uint32_t expert = 0xFFFFFFFFu - best_lo;
                if (expert >= experts)
                    expert = 0; // only when every remaining key is NaN
                if (lane == 0)
                {
                    records[expert] = 0ull;
                    out_expert[r] = expert;
                }
                __syncwarp();
            }
        }
        if (token_failed)
            continue;
        __syncwarp();
        __threadfence_block();
        // rank-order sequential sum of the unbiased scores (:131-133)
        for (uint32_t base = 0; base < top_k; base += 32)
        {
            const uint32_t r = base + lane;
            const float score = (r < top_k) ? scores[out_expert[r]] : 0.0f;
            const uint32_t steps = min(32u, top_k - base);
            for (uint32_t j = 0; j < steps; ++j)
                chosen_total = __fadd_rn(chosen_total, __shfl_sync(kFullMask, score, j));
        }
        if (renormalize && chosen_total <= 0.0f)
        {
            if (lane == 0)
                report_error(error_word, 1, token, 103);
            continue;
        }
        for (uint32_t r = lane; r < top_k; r += 32)
        {
            const uint32_t expert = out_expert[r];
            const float score = scores[expert];
            const float weight = __fmul_rn(renormalize ? __fdiv_rn(score, chosen_total) : score, a.options.routed_scaling_factor);
            out_weight[r] = weight;
            atomicAdd(&expert_counts[expert], 1u);
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(1024) router_offsets_kernel(uint32_t experts, uint32_t* expert_counts, uint32_t* expert_offsets,
                                                              unsigned long long* error_word, int32_t* plan_status)
{
    __shared__ uint32_t warp_sums[32];
    __shared__ uint32_t carry;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    if (tid == 0)
        carry = 0;
    __syncthreads();
    for (uint32_t base = 0; base < experts; base += 1024)
    {
        const uint32_t e = base + tid;
        const uint32_t value = (e < experts) ? expert_counts[e] : 0u;
        uint32_t inclusive = value;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1)
        {
            const uint32_t other = __shfl_up_sync(kFullMask, inclusive, offset);
            if (lane >= offset)
                inclusive += other;
        }
        if (lane == 31)
            warp_sums[warp] = inclusive;
        __syncthreads();
        if (warp == 0)
        {
            const uint32_t sum = warp_sums[lane];
            uint32_t scan = sum;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1)
            {
                const uint32_t other = __shfl_up_sync(kFullMask, scan, offset);
                if (lane >= offset)
                    scan += other;
            }
            warp_sums[lane] = scan - sum;
        }
        __syncthreads();
        const uint32_t exclusive = carry + warp_sums[warp] + inclusive - value;
        if (e < experts)
        {
            expert_offsets[e] = exclusive;
            expert_counts[e] = 0; // ready for the next call
        }
        __syncthreads();
        if (tid == 1023)
            carry = exclusive + value;
        __syncthreads();
    }
    if (tid == 0)
    {
        expert_offsets[experts] = carry;
        const unsigned long long word = *error_word;
        plan_status[0] = (word == ~0ull) ? 0 : static_cast<int32_t>(word & 0xFFu);
        *error_word = ~0ull;
    }
}

__global__ void __launch_bounds__(256) router_group_kernel(const RouterArgs a)
{
    __shared__ uint32_t warp_counts[8];
    __shared__ uint32_t running;
    const uint32_t expert = blockIdx.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t total = a.token_count * a.options.top_k;
    const uint32_t begin = a.expert_offsets[expert];
    if (a.plan_status[0] != 0 || a.expert_offsets[expert + 1] == begin)
        return; // a failed call leaves no plan; an idle expert has nothing to place
    if (tid == 0)
        running = 0;
    __syncthreads();
    for (uint32_t base = 0; base < total; base += 256)
    {
        const uint32_t i = base + tid;
        const bool match = (i < total) && (a.selected_expert[i] == expert);
        const unsigned voters = __ballot_sync(kFullMask, match);
        if (lane == 0)
            warp_counts[warp] = __popc(voters);
        __syncthreads();
        uint32_t before = running;
        for (int w = 0; w < warp; ++w)
            before += warp_counts[w];
        if (match)
        {
            const uint32_t slot = begin + before + __popc(voters & ((1u << lane) - 1u));
            a.route_token[slot] = i / a.options.top_k;
            a.route_rank[slot] = i % a.options.top_k;
            a.route_weight[slot] = a.selected_weight[i];
        }
        __syncthreads();
        if (tid == 0)
        {
            uint32_t sum = running;
            for (int w = 0; w < 8; ++w)
                sum += warp_counts[w];
            running = sum;
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256) regroup_gather_kernel(const float* hidden, uint32_t columns, const uint32_t* route_token, uint32_t route_count,
                                                             float* gathered, int vectorised)
{
    // one warp per route row keeps each copy a run of full 128-byte lines
    const uint32_t warps_per_block = 256 / 32;
    const int lane = threadIdx.x & 31;
    for (uint32_t route = blockIdx.x * warps_per_block + (threadIdx.x >> 5); route < route_count; route += gridDim.x * warps_per_block)
    {
        const float* source = hidden + static_cast<size_t>(route_token[route]) * columns;
        float* target = gathered + static_cast<size_t>(route) * columns;
        if (vectorised)
        {
            const float4* source4 = reinterpret_cast<const float4*>(source);
            float4* target4 = reinterpret_cast<float4*>(target);
            for (uint32_t c = lane; c < columns / 4; c += 32)
                target4[c] = source4[c];
        }
        else
        {
            for (uint32_t c = lane; c < columns; c += 32)
                target[c] = source[c];
        }
    }
}

} // namespace

cudaError_t launch_router_dispatch_kernels(const RouterArgs& args, uint32_t* expert_counts, unsigned long long* error_word, cudaStream_t stream)
{
    const uint32_t experts = args.options.expert_count;
    const size_t shared_bytes = static_cast<size_t>(kRouteWarps) * experts * (sizeof(float) + sizeof(uint64_t));
    static size_t configured_bytes = 48 * 1024;
    if (shared_bytes > configured_bytes)
    {
        cudaError_t status = cudaFuncSetAttribute(router_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared_bytes));
        if (status != cudaSuccess)
            return status;
        configured_bytes = shared_bytes;
    }
    const uint32_t blocks_needed = (args.token_count + kRouteWarps - 1) / kRouteWarps;
    const uint32_t grid = blocks_needed < 148u * 8u ? blocks_needed : 148u * 8u;
    router_select_kernel<<<grid, kRouteThreads, shared_bytes, stream>>>(args, expert_counts, error_word);
    router_offsets_kernel<<<1, 1024, 0, stream>>>(experts, expert_counts, args.expert_offsets, error_word, args.plan_status);
    router_group_kernel<<<experts, 256, 0, stream>>>(args);
    return cudaGetLastError();
}

cudaError_t launch_regroup_gather(const float* hidden, uint32_t columns, const uint32_t* route_token, uint32_t route_count, float* gathered,
                                  cudaStream_t stream)
{
    if (route_count == 0 || columns == 0)
        return cudaSuccess;
    const int vectorised = (columns % 4 == 0) && ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(gathered)) % 16 == 0);
    const uint32_t blocks_needed = (route_count + 7) / 8;
    const uint32_t grid = blocks_needed < 148u * 16u ? blocks_needed : 148u * 16u;
    regroup_gather_kernel<<<grid, 256, 0, stream>>>(hidden, columns, route_token, route_count, gathered, vectorised);
    return cudaGetLastError();
}


// ---- router dispatch without any allocation ------------------------------------
//
// Some hosts of this library may not call cudaMalloc at the point where they
// route tokens: a serving engine that has handed every byte of device memory
// to its own planner or pool up front (so a late allocation either fails or
// breaks the planner's accounting), or a decode loop that cannot afford the
// device-wide synchronisation an allocation may imply.  moe_router_dispatch
// grows its scratch on demand and so does not suit them.  This variant keeps
// the scratch the three router kernels need — the per-route (expert, weight)
// pairs, the per-expert counters and the error word — in one fixed array that
// lives in the library's device image.  Every GPU that loads the library
// carries these MOE_ROUTER_STATIC_SCRATCH_BYTES until the process exits.

namespace {

struct StaticRouterScratch
{
    unsigned long long error_word;
    uint32_t expert_counts[MOE_ROUTER_STATIC_MAX_EXPERTS];
    uint32_t selected_expert[MOE_ROUTER_STATIC_MAX_ROUTES];
    float selected_weight[MOE_ROUTER_STATIC_MAX_ROUTES];
};
static_assert(sizeof(StaticRouterScratch) <= MOE_ROUTER_STATIC_SCRATCH_BYTES, "scratch layout outgrew the documented size");

// Device storage.  In host code this name is only a handle for the runtime's
// symbol lookup, never a pointer a kernel may be given.
static __device__ __align__(256) unsigned char g_router_static_scratch[MOE_ROUTER_STATIC_SCRATCH_BYTES];

constexpr int kStaticMaxDevices = 64;
// Device address of the array, looked up once per device ordinal.
void* g_router_static_address[kStaticMaxDevices] = {};

// The array keeps whatever the previous call left in it: counters and the
// error word must be back at their start values before the select kernel runs.
__global__ void router_static_reset_kernel(StaticRouterScratch* scratch, uint32_t experts)
{
    for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < experts; e += gridDim.x * blockDim.x)
        scratch->expert_counts[e] = 0;
    if (blockIdx.x == 0 && threadIdx.x == 0)
        scratch->error_word = ~0ull;
}

void describe(char* text, size_t capacity, const char* message)
{
    if (text != nullptr && capacity > 0)
        snprintf(text, capacity, "%s", message);
}

} // namespace

} // namespace moe

extern "C" int moe_router_dispatch_static(void* stream_handle, const float* router_logits, uint32_t token_count,
                                          const moe_router_options* options, uint32_t* expert_offsets, uint32_t* route_token,
                                          uint32_t* route_rank, float* route_weight, int32_t* plan_status, char* error_text,
                                          size_t error_capacity)
{
    using namespace moe;
    describe(error_text, error_capacity, "");
    const int precheck = moe_router_check_options(token_count, options);
    if (precheck != 0)
    {
        describe(error_text, error_capacity, moe_router_status_message(precheck));
        return moe_router_status_error_code(precheck);
    }
    if (router_logits == nullptr || expert_offsets == nullptr || route_token == nullptr || route_rank == nullptr || route_weight == nullptr ||
        plan_status == nullptr)
    {
        describe(error_text, error_capacity, "router buffers must not be null");
        return MOE_STATUS_INVALID_ARGUMENT;
    }
    const uint64_t routes = static_cast<uint64_t>(token_count) * options->top_k;
    if (routes > MOE_ROUTER_STATIC_MAX_ROUTES)
    {
        describe(error_text, error_capacity,
                 "token_count * top_k exceeds MOE_ROUTER_STATIC_MAX_ROUTES, the fixed scratch of moe_router_dispatch_static; "
                 "split the tokens over several calls or use moe_router_dispatch");
        return MOE_STATUS_INVALID_ARGUMENT;
    }
    if (options->expert_count > MOE_ROUTER_STATIC_MAX_EXPERTS)
    {
        describe(error_text, error_capacity, "expert_count exceeds MOE_ROUTER_STATIC_MAX_EXPERTS, the fixed scratch of moe_router_dispatch_static");
        return MOE_STATUS_INVALID_ARGUMENT;
    }
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess || device < 0 || device >= kStaticMaxDevices)
    {
        describe(error_text, error_capacity, status != cudaSuccess ? cudaGetErrorString(status) : "device ordinal beyond the static table");
        return MOE_STATUS_CUDA_ERROR;
    }
    if (g_router_static_address[device] == nullptr)
    {
        // first call on this device (it is the current one): resolve the array's device address
        void* address = nullptr;
        status = cudaGetSymbolAddress(&address, g_router_static_scratch);
        if (status != cudaSuccess || address == nullptr)
        {
            describe(error_text, error_capacity, status != cudaSuccess ? cudaGetErrorString(status) : "symbol lookup returned no address");
            return MOE_STATUS_CUDA_ERROR;
        }
        g_router_static_address[device] = address;
    }
    StaticRouterScratch* scratch = static_cast<StaticRouterScratch*>(g_router_static_address[device]);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);

    const uint32_t experts = options->expert_count;
    router_static_reset_kernel<<<(experts + 255) / 256, 256, 0, stream>>>(scratch, experts);
    status = cudaGetLastError();
    if (status != cudaSuccess)
    {
        describe(error_text, error_capacity, cudaGetErrorString(status));
        return MOE_STATUS_CUDA_ERROR;
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
    args.selected_expert = scratch->selected_expert; // address arithmetic on the device pointer only; nothing is read here
    args.selected_weight = scratch->selected_weight;
    status = launch_router_dispatch_kernels(args, scratch->expert_counts, &scratch->error_word, stream);
    if (status != cudaSuccess)
    {
        describe(error_text, error_capacity, cudaGetErrorString(status));
        return MOE_STATUS_CUDA_ERROR;
    }
    return MOE_STATUS_OK;
}

namespace moe {
} // namespace moe
