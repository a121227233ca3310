// MoE router: scoring, stable Top-K, weights and grouping by expert.
// Replaces ExpertDispatcher::dispatch (src/graph/expert_dispatcher.cpp:79-158)
// and gather_tokens (src/engine/cpu_executor.cpp:635-642).
//
// The grouping is a stable counting sort of the routes by expert:
// Kernel 1, select (one warp per token, a block owns a contiguous run of
//   tokens): scores in the reference's arithmetic (softmax with an index-order
//   sequential sum, sigmoid, sqrt-softplus; expert_dispatcher.cpp:24-59),
//   selection key = score + bias, stable Top-K on (key descending, expert id
//   ascending) records — the record/ordering primitive the sampler uses; k
//   rounds of a warp arg-max for narrow routers, a radix select of the k
//   survivors first for wide ones — then the rank-order sequential sum of the
//   unbiased scores and the weights (:131-144).  Each block counts its routes
//   per expert in shared memory and writes the counts to its column of a
//   [expert][block] table: no global atomics, so the result is deterministic.
// Kernel 2, scan (one warp per expert): exclusive prefix of the expert's counts
//   over the blocks, its total; the block that finishes last turns the totals
//   into CSR offsets and the call status.
// Kernel 3, place (one warp per block of kernel 1): walks the block's routes in
//   (token, rank) order; a route's slot is its expert's offset + the routes of
//   earlier blocks + its rank among the block's earlier routes of that expert
//   (warp match), which is the order the reference appends them in (:146-157).

#include <cstdio>

#include "moe_common.cuh"
#include "moe_internal.h"

namespace moe {

namespace {

constexpr int kRouteThreads = 128;
constexpr int kRouteWarps = kRouteThreads / 32;
constexpr uint32_t kNarrowExperts = 1024; // above this, or above kNarrowTopK, the survivors are radix-selected first
constexpr uint32_t kNarrowTopK = 16;

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

// Keeps the k largest of records[0..n) (unique, non-zero, 0 < k < n) in
// records[0..k), in no particular order.  One warp; `hist` is 256 words of that
// warp's shared memory.  Digits of 8 bits from the highest bit on which the
// records differ, early exit when a bucket boundary falls on k.
__device__ __forceinline__ void warp_radix_select(uint64_t* records, uint32_t n, uint32_t k, uint32_t* hist)
{
    const int lane = threadIdx.x & 31;
    uint64_t any_bits = 0, all_bits = ~0ull;
    for (uint32_t i = lane; i < n; i += 32)
    {
        any_bits |= records[i];
        all_bits &= records[i];
    }
    any_bits = warp_or_u64(any_bits);
    all_bits = warp_and_u64(all_bits);
    const uint64_t varying = any_bits ^ all_bits;
    int high = 63 - __clzll(static_cast<long long>(varying | 1ull));
    uint64_t prefix_mask = (high >= 63) ? 0ull : (~0ull << (high + 1));
    uint64_t prefix_value = all_bits & prefix_mask;
    uint32_t remaining = k;
    int low = 0;
    for (;;)
    {
        low = (high >= 7) ? (high - 7) : 0;
        const uint32_t digit_mask = (1u << (high - low + 1)) - 1u;
#pragma unroll
        for (int b = 0; b < 8; ++b)
            hist[lane * 8 + b] = 0;
        __syncwarp();
        for (uint32_t i = lane; i < n; i += 32)
        {
            const uint64_t record = records[i];
            if ((record & prefix_mask) == prefix_value)
                atomicAdd(&hist[static_cast<uint32_t>(record >> low) & digit_mask], 1u);
        }
        __syncwarp();
        // lane owns bins [8*lane, 8*lane+8); walk from the top bin down
        uint32_t bins[8];
        uint32_t lane_total = 0;
#pragma unroll
        for (int b = 0; b < 8; ++b)
        {
            bins[b] = hist[lane * 8 + b];
            lane_total += bins[b];
        }
        uint32_t suffix = lane_total; // inclusive sum over lanes >= this one
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1)
        {
            const uint32_t other = __shfl_down_sync(kFullMask, suffix, offset);
            if (lane + offset < 32)
                suffix += other;
        }
        const unsigned reach = __ballot_sync(kFullMask, suffix >= remaining);
        const int owner = 31 - __clz(static_cast<int>(reach));
        uint32_t bucket = 0, bucket_count = 0, above = 0;
        if (lane == owner)
        {
            uint32_t cumulative = suffix - lane_total;
#pragma unroll
            for (int b = 7; b >= 0; --b)
            {
                if (cumulative + bins[b] >= remaining)
                {
                    bucket = lane * 8 + b;
                    bucket_count = bins[b];
                    above = cumulative;
                    break;
                }
                cumulative += bins[b];
            }
        }
        bucket = __shfl_sync(kFullMask, bucket, owner);
        bucket_count = __shfl_sync(kFullMask, bucket_count, owner);
        above = __shfl_sync(kFullMask, above, owner);
        remaining -= above;
        prefix_value |= static_cast<uint64_t>(bucket) << low;
        prefix_mask |= static_cast<uint64_t>(digit_mask) << low;
        __syncwarp();
        if (bucket_count == remaining || low == 0)
            break;
        high = low - 1;
    }
    // everything whose high bits (down to `low`) reach the threshold's is kept: exactly k records
    const uint64_t threshold = prefix_value >> low;
    uint32_t kept = 0;
    for (uint32_t base = 0; base < n; base += 32)
    {
        const uint32_t i = base + lane;
        const uint64_t record = (i < n) ? records[i] : 0ull;
        const bool keep = (i < n) && ((record >> low) >= threshold);
        const unsigned voters = __ballot_sync(kFullMask, keep);
        // slots below `base` have all been read, and kept <= base: the write never overtakes a read
        if (keep)
            records[kept + __popc(voters & ((1u << lane) - 1u))] = record;
        kept += __popc(voters);
        __syncwarp();
    }
}

__global__ void __launch_bounds__(kRouteThreads) router_select_kernel(const RouterArgs a, unsigned long long* error_word)
{
    extern __shared__ __align__(16) unsigned char shared_raw[];
    const uint32_t experts = a.options.expert_count;
    const uint32_t top_k = a.options.top_k;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    // shared: scores [warps][experts] | records [warps][experts] | block counts [experts] | radix bins [warps][256]
    float* scores = reinterpret_cast<float*>(shared_raw) + static_cast<size_t>(warp) * experts;
    uint64_t* records = reinterpret_cast<uint64_t*>(shared_raw + sizeof(float) * experts * kRouteWarps) + static_cast<size_t>(warp) * experts;
    uint32_t* block_counts = reinterpret_cast<uint32_t*>(shared_raw + (sizeof(float) + sizeof(uint64_t)) * experts * kRouteWarps);
    uint32_t* radix_bins = block_counts + experts + warp * 256;
    const bool renormalize = (a.options.flags & MOE_ROUTER_FLAG_NORMALIZE_TOPK) != 0 || a.options.normalization == 1;
    const bool wide = experts > kNarrowExperts || top_k > kNarrowTopK;

    for (uint32_t e = threadIdx.x; e < experts; e += kRouteThreads)
        block_counts[e] = 0;
    __syncthreads();

    const uint32_t token_begin = blockIdx.x * a.tokens_per_block;
    const uint32_t token_end = min(a.token_count, token_begin + a.tokens_per_block);
    for (uint32_t token = token_begin + warp; token < token_end; token += kRouteWarps)
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
            bool nan_key = false;
            for (uint32_t e = lane; e < experts; e += 32)
            {
                const float key = (a.options.selection_bias != nullptr) ? __fadd_rn(scores[e], a.options.selection_bias[e]) : scores[e];
                // NaN keys never win a `>` compare in the reference; rank them last
                records[e] = (key == key) ? make_record(ordered_key(key), e) : 0ull;
                nan_key |= !(key == key);
            }
            __syncwarp();
            uint32_t pool = experts; // records the arg-max rounds look at
            if (wide && top_k < experts && !__any_sync(kFullMask, nan_key))
            {
                warp_radix_select(records, experts, top_k, radix_bins);
                pool = top_k;
            }
            for (uint32_t r = 0; r < top_k; ++r)
            {
                uint64_t best = 0ull;
                uint32_t best_slot = 0;
                for (uint32_t i = lane; i < pool; i += 32)
                {
                    const uint64_t record = records[i];
                    if (record > best)
                    {
                        best = record;
                        best_slot = i;
                    }
                }
                const uint32_t best_hi = __reduce_max_sync(kFullMask, static_cast<uint32_t>(best >> 32));
                const uint32_t candidate_lo = (static_cast<uint32_t>(best >> 32) == best_hi) ? static_cast<uint32_t>(best) : 0u;
                const uint32_t best_lo = __reduce_max_sync(kFullMask, candidate_lo);
                const bool mine = best != 0ull && static_cast<uint32_t>(best >> 32) == best_hi && static_cast<uint32_t>(best) == best_lo;
                uint32_t expert = 0xFFFFFFFFu - best_lo;
                if (expert >= experts)
                    expert = 0; // only when every remaining key is NaN
                if (mine)
                    records[best_slot] = 0ull; // records are unique: exactly one lane owns the winner
                if (lane == 0)
                    out_expert[r] = expert;
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
            atomicAdd(&block_counts[expert], 1u);
        }
        __syncwarp();
    }
    __syncthreads();
    // this block's column of the [expert][block] table
    for (uint32_t e = threadIdx.x; e < experts; e += kRouteThreads)
        a.block_counts[static_cast<size_t>(e) * gridDim.x + blockIdx.x] = block_counts[e];
}

// One warp per expert: exclusive prefix of its per-block counts (in place) and
// its total.  The block that finishes last scans the totals into CSR offsets
// and publishes the call status.
__global__ void __launch_bounds__(256) router_scan_kernel(uint32_t experts, uint32_t blocks, uint32_t* block_counts, uint32_t* expert_counts,
                                                          uint32_t* expert_offsets, uint32_t* scan_done, unsigned long long* error_word,
                                                          int32_t* plan_status)
{
    __shared__ uint32_t warp_sums[8];
    __shared__ uint32_t carry;
    __shared__ uint32_t is_last;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t expert = blockIdx.x * 8u + warp;
    if (expert < experts)
    {
        uint32_t* column = block_counts + static_cast<size_t>(expert) * blocks;
        uint32_t running = 0;
        for (uint32_t base = 0; base < blocks; base += 32)
        {
            const uint32_t b = base + lane;
            const uint32_t value = (b < blocks) ? column[b] : 0u;
            uint32_t inclusive = value;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1)
            {
                const uint32_t other = __shfl_up_sync(kFullMask, inclusive, offset);
                if (lane >= offset)
                    inclusive += other;
            }
            if (b < blocks)
                column[b] = running + inclusive - value;
            running += __shfl_sync(kFullMask, inclusive, 31);
        }
        if (lane == 0)
            expert_counts[expert] = running;
    }
    __syncthreads();
    if (tid == 0)
    {
        __threadfence();
        is_last = (atomicAdd(scan_done, 1u) == gridDim.x - 1u) ? 1u : 0u;
        carry = 0;
    }
    __syncthreads();
    if (is_last == 0u)
        return;
    __threadfence();
    for (uint32_t base = 0; base < experts; base += 256)
    {
        const uint32_t e = base + tid;
        const uint32_t value = (e < experts) ? __ldcg(expert_counts + e) : 0u;
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
        uint32_t before = carry;
        for (int w = 0; w < warp; ++w)
            before += warp_sums[w];
        if (e < experts)
            expert_offsets[e] = before + inclusive - value;
        __syncthreads();
        if (tid == 255)
            carry = before + inclusive;
        __syncthreads();
    }
    if (tid == 0)
    {
        expert_offsets[experts] = carry;
        const unsigned long long word = *error_word;
        plan_status[0] = (word == ~0ull) ? 0 : static_cast<int32_t>(word & 0xFFu);
        *error_word = ~0ull; // ready for the next call
        *scan_done = 0;
    }
}

// One warp per block of the select kernel, walking that block's routes in
// (token, rank) order, 32 at a time.
__global__ void __launch_bounds__(kRouteThreads) router_place_kernel(const RouterArgs a, uint32_t blocks)
{
    const int lane = threadIdx.x & 31;
    const uint32_t segment = blockIdx.x * kRouteWarps + (threadIdx.x >> 5);
    if (segment >= blocks || a.plan_status[0] != 0)
        return; // a failed call leaves no plan
    const uint32_t top_k = a.options.top_k;
    const uint32_t token_begin = segment * a.tokens_per_block;
    const uint32_t token_end = min(a.token_count, token_begin + a.tokens_per_block);
    const uint32_t route_begin = token_begin * top_k;
    const uint32_t route_end = token_end * top_k;
    const unsigned lanes_below = (1u << lane) - 1u;
    for (uint32_t base = route_begin; base < route_end; base += 32)
    {
        const uint32_t i = base + lane;
        const bool live = i < route_end;
        const uint32_t expert = live ? a.selected_expert[i] : 0xFFFFFFFFu;
        const unsigned peers = __match_any_sync(kFullMask, expert);
        const int leader = __ffs(peers) - 1;
        uint32_t before = 0;
        if (live && lane == leader)
        {
            // routes of this expert placed so far: earlier blocks (the scan's prefix) + earlier rounds of this warp
            before = atomicAdd(a.block_counts + static_cast<size_t>(expert) * blocks + segment, static_cast<uint32_t>(__popc(peers)));
        }
        before = __shfl_sync(kFullMask, before, leader);
        if (live)
        {
            const uint32_t slot = a.expert_offsets[expert] + before + __popc(peers & lanes_below);
            a.route_token[slot] = i / top_k;
            a.route_rank[slot] = i % top_k;
            a.route_weight[slot] = a.selected_weight[i];
        }
        __syncwarp(); // rounds stay in order: the next round's leader may be another lane
    }
}

__global__ void __launch_bounds__(256) regroup_gather_kernel(const float* hidden, uint32_t token_count, uint32_t columns, const uint32_t* route_token,
                                                             uint32_t route_count, float* gathered, int32_t* out_of_range, int vectorised)
{
    // one warp per route row keeps each copy a run of full 128-byte lines
    const uint32_t warps_per_block = 256 / 32;
    const int lane = threadIdx.x & 31;
    for (uint32_t route = blockIdx.x * warps_per_block + (threadIdx.x >> 5); route < route_count; route += gridDim.x * warps_per_block)
    {
        const uint32_t token = route_token[route];
        // a token index beyond the hidden matrix is never dereferenced: its row is zero-filled and the call flagged
        const bool valid = token < token_count;
        if (!valid && lane == 0)
            *out_of_range = 1;
        const float* source = hidden + static_cast<size_t>(valid ? token : 0u) * columns;
        float* target = gathered + static_cast<size_t>(route) * columns;
        if (vectorised)
        {
            const float4* source4 = reinterpret_cast<const float4*>(source);
            float4* target4 = reinterpret_cast<float4*>(target);
            // eight 16-byte loads in flight per lane; the copies leave with a streaming store so that the
            // hidden rows (read once per route of their token) stay in L2
            const uint32_t vectors = columns / 4;
            const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            uint32_t c = lane;
            for (; c + 7u * 32u < vectors; c += 8u * 32u)
            {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    v[u] = valid ? __ldg(source4 + c + 32u * u) : zero;
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    __stcs(target4 + c + 32u * u, v[u]);
            }
            for (; c < vectors; c += 32)
                __stcs(target4 + c, valid ? __ldg(source4 + c) : zero);
        }
        else
        {
            for (uint32_t c = lane; c < columns; c += 32)
                target[c] = valid ? source[c] : 0.0f;
        }
    }
}

} // namespace

cudaError_t launch_router_dispatch_kernels(const RouterArgs& caller_args, uint32_t* expert_counts, uint32_t* scan_done, unsigned long long* error_word,
                                           cudaStream_t stream)
{
    RouterArgs args = caller_args;
    const uint32_t experts = args.options.expert_count;
    static_assert(kRouteWarps == 4, "router_partition_host assumes four warps per block");
    const RouterPartition part = router_partition_host(args.token_count, experts);
    args.tokens_per_block = part.tokens_per_block;
    const size_t shared_bytes = static_cast<size_t>(kRouteWarps) * experts * (sizeof(float) + sizeof(uint64_t)) + sizeof(uint32_t) * experts +
                                sizeof(uint32_t) * 256u * kRouteWarps;
    static SharedOptIn opt_in;
    if (shared_bytes > 48u * 1024u)
    {
        if (cudaError_t status = opt_in_shared(opt_in, router_select_kernel, shared_bytes))
            return status;
    }
    router_select_kernel<<<part.blocks, kRouteThreads, shared_bytes, stream>>>(args, error_word);
    router_scan_kernel<<<(experts + 7u) / 8u, 256, 0, stream>>>(experts, part.blocks, args.block_counts, expert_counts, args.expert_offsets, scan_done,
                                                                  error_word, args.plan_status);
    router_place_kernel<<<(part.blocks + kRouteWarps - 1u) / kRouteWarps, kRouteThreads, 0, stream>>>(args, part.blocks);
    return cudaGetLastError();
}

cudaError_t launch_regroup_gather(const float* hidden, uint32_t token_count, uint32_t columns, const uint32_t* route_token, uint32_t route_count,
                                  float* gathered, int32_t* out_of_range, cudaStream_t stream)
{
    if (route_count == 0 || columns == 0)
        return cudaSuccess;
    const int vectorised = (columns % 4 == 0) && ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(gathered)) % 16 == 0);
    const uint32_t blocks_needed = (route_count + 7) / 8;
    const uint32_t grid = blocks_needed < 148u * 16u ? blocks_needed : 148u * 16u;
    regroup_gather_kernel<<<grid, 256, 0, stream>>>(hidden, token_count, columns, route_token, route_count, gathered, out_of_range, vectorised);
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
// pairs, the per-expert and per-block counters and the error word — in one fixed array that
// lives in the library's device image.  Every GPU that loads the library
// carries these MOE_ROUTER_STATIC_SCRATCH_BYTES until the process exits.

namespace {

struct StaticRouterScratch
{
    unsigned long long error_word;
    uint32_t expert_counts[MOE_ROUTER_STATIC_MAX_EXPERTS];
    uint32_t selected_expert[MOE_ROUTER_STATIC_MAX_ROUTES];
    float selected_weight[MOE_ROUTER_STATIC_MAX_ROUTES];
    uint32_t scan_done;
    uint32_t block_counts[MOE_ROUTER_BLOCK_TABLE_ENTRIES];
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
__global__ void router_static_reset_kernel(StaticRouterScratch* scratch)
{
    // the per-expert counts and the [expert][block] table are fully rewritten by every call
    scratch->error_word = ~0ull;
    scratch->scan_done = 0;
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

    router_static_reset_kernel<<<1, 1, 0, stream>>>(scratch);
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
    args.block_counts = scratch->block_counts;
    status = launch_router_dispatch_kernels(args, scratch->expert_counts, &scratch->scan_done, &scratch->error_word, stream);
    if (status != cudaSuccess)
    {
        describe(error_text, error_capacity, cudaGetErrorString(status));
        return MOE_STATUS_CUDA_ERROR;
    }
    return MOE_STATUS_OK;
}

namespace moe {
} // namespace moe
