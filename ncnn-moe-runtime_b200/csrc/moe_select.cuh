// Block-wide selection primitives over candidate records held in shared
// memory: radix select of the k largest records (stable: the token index is
// part of the record, so equal logits resolve to the lowest index), predicate
// compaction, and a bitonic sort used only on the final <= few thousand
// survivors that the sequential softmax / Top-P arithmetic must walk in rank
// order.  Replaces the full std::stable_sort of src/engine/session.cpp:80-82
// and the insertion Top-K of src/graph/expert_dispatcher.cpp:61-77.
#pragma once

#include "moe_common.cuh"

namespace moe {

template<int kThreads>
struct SelectShared
{
    uint32_t hist[256];
    uint64_t reduce_or[kThreads / 32];
    uint64_t reduce_and[kThreads / 32];
    uint32_t bucket;
    uint32_t bucket_count;
    uint32_t above;
    uint32_t out_count;
    unsigned long long out_min;
};

// Keeps the k largest of records[0..n) (n > k >= 1, n <= kItems * kThreads) in
// records[0..k), in no particular order.  Returns the smallest kept record.
// All threads of the block must call it; ends with a barrier.
template<int kThreads, int kItems>
__device__ __noinline__ uint64_t block_radix_select(uint64_t* records, uint32_t n, uint32_t k, SelectShared<kThreads>& sh)
{
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

    const int used = static_cast<int>((n + kThreads - 1) / kThreads); // item slots that hold anything
    uint64_t item[kItems];
    uint64_t any_bits = 0;
    uint64_t all_bits = ~0ull;
#pragma unroll
    for (int j = 0; j < kItems; ++j)
    {
        if (j >= used)
            break;
        const uint32_t i = tid + j * kThreads;
        item[j] = (i < n) ? records[i] : 0ull;
        if (i < n)
        {
            any_bits |= item[j];
            all_bits &= item[j];
        }
    }
    any_bits = warp_or_u64(any_bits);
    all_bits = warp_and_u64(all_bits);
    if (lane == 0)
    {
        sh.reduce_or[warp] = any_bits;
        sh.reduce_and[warp] = all_bits;
    }
    __syncthreads();
    any_bits = 0;
    all_bits = ~0ull;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w)
    {
        any_bits |= sh.reduce_or[w];
        all_bits &= sh.reduce_and[w];
    }
    // Bits on which at least two records differ.  Records are unique (the
    // token index is in the low word), so with n > 1 this is never zero.
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
        sh.hist[tid & 255] = 0; // kThreads >= 256
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kItems; ++j)
        {
            if (j >= used)
                break;
            const uint32_t i = tid + j * kThreads;
            const bool live = (i < n) && ((item[j] & prefix_mask) == prefix_value);
            const uint32_t digit = live ? (static_cast<uint32_t>(item[j] >> low) & digit_mask) : 0xFFFFFFFFu;
            const unsigned peers = __match_any_sync(kFullMask, digit);
            if (live && lane == (__ffs(peers) - 1))
                atomicAdd(&sh.hist[digit], __popc(peers));
        }
        __syncthreads();
        if (warp == 0)
        {
            // lane owns bins [8*lane, 8*lane+8); walk from the top bin down
            uint32_t bins[8];
            uint32_t lane_total = 0;
#pragma unroll
            for (int b = 0; b < 8; ++b)
            {
                bins[b] = sh.hist[lane * 8 + b];
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
            if (lane == owner)
            {
                uint32_t cumulative = suffix - lane_total;
#pragma unroll
                for (int b = 7; b >= 0; --b)
                {
                    if (cumulative + bins[b] >= remaining)
                    {
                        sh.bucket = lane * 8 + b;
                        sh.bucket_count = bins[b];
                        sh.above = cumulative;
                        break;
                    }
                    cumulative += bins[b];
                }
            }
        }
        __syncthreads();
        const uint32_t bucket = sh.bucket;
        const uint32_t bucket_count = sh.bucket_count;
        remaining -= sh.above;
        prefix_value |= static_cast<uint64_t>(bucket) << low;
        prefix_mask |= static_cast<uint64_t>(digit_mask) << low;
        if (bucket_count == remaining || low == 0)
            break;
        high = low - 1;
    }

    // Everything whose high bits (down to `low`) are >= the threshold's is kept.
    if (tid == 0)
    {
        sh.out_count = 0;
        sh.out_min = ~0ull;
    }
    __syncthreads();
    const uint64_t threshold = prefix_value >> low;
    uint64_t local_min = ~0ull;
#pragma unroll
    for (int j = 0; j < kItems; ++j)
    {
        if (j >= used)
            break;
        const uint32_t i = tid + j * kThreads;
        const bool keep = (i < n) && ((item[j] >> low) >= threshold);
        const unsigned voters = __ballot_sync(kFullMask, keep);
        if (voters != 0)
        {
            uint32_t base = 0;
            if (lane == (__ffs(voters) - 1))
                base = atomicAdd(&sh.out_count, __popc(voters));
            base = __shfl_sync(kFullMask, base, __ffs(voters) - 1);
            if (keep)
            {
                records[base + __popc(voters & ((1u << lane) - 1u))] = item[j];
                local_min = (item[j] < local_min) ? item[j] : local_min;
            }
        }
    }
    // warp min of a 64-bit value
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
    {
        const uint64_t other = __shfl_xor_sync(kFullMask, local_min, offset);
        local_min = (other < local_min) ? other : local_min;
    }
    if (lane == 0 && local_min != ~0ull)
        atomicMin(&sh.out_min, static_cast<unsigned long long>(local_min));
    __syncthreads();
    const uint64_t result = sh.out_min;
    __syncthreads(); // the next user of `sh` may overwrite out_min at once
    return result;
}

// Smallest record of records[0..n), n >= 1.  Ends with a barrier.
template<int kThreads>
__device__ __noinline__ uint64_t block_min_record(const uint64_t* records, uint32_t n, SelectShared<kThreads>& sh)
{
    const int tid = threadIdx.x;
    if (tid == 0)
        sh.out_min = ~0ull;
    __syncthreads();
    uint64_t local_min = ~0ull;
    for (uint32_t i = tid; i < n; i += kThreads)
        local_min = (records[i] < local_min) ? records[i] : local_min;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
    {
        const uint64_t other = __shfl_xor_sync(kFullMask, local_min, offset);
        local_min = (other < local_min) ? other : local_min;
    }
    if ((tid & 31) == 0 && local_min != ~0ull)
        atomicMin(&sh.out_min, static_cast<unsigned long long>(local_min));
    __syncthreads();
    const uint64_t result = sh.out_min;
    __syncthreads(); // the next user of `sh` may overwrite out_min at once
    return result;
}

// Keeps the records for which keep(record) holds, in records[0..result).
// n <= kItems * kThreads.  Ends with a barrier.
template<int kThreads, int kItems, typename Keep>
__device__ __forceinline__ uint32_t block_compact(uint64_t* records, uint32_t n, SelectShared<kThreads>& sh, Keep keep_record)
{
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int used = static_cast<int>((n + kThreads - 1) / kThreads);
    uint64_t item[kItems];
#pragma unroll
    for (int j = 0; j < kItems; ++j)
    {
        if (j >= used)
            break;
        const uint32_t i = tid + j * kThreads;
        item[j] = (i < n) ? records[i] : 0ull;
    }
    if (tid == 0)
        sh.out_count = 0;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kItems; ++j)
    {
        if (j >= used)
            break;
        const uint32_t i = tid + j * kThreads;
        const bool keep = (i < n) && keep_record(item[j]);
        const unsigned voters = __ballot_sync(kFullMask, keep);
        if (voters != 0)
        {
            uint32_t base = 0;
            if (lane == (__ffs(voters) - 1))
                base = atomicAdd(&sh.out_count, __popc(voters));
            base = __shfl_sync(kFullMask, base, __ffs(voters) - 1);
            if (keep)
                records[base + __popc(voters & ((1u << lane) - 1u))] = item[j];
        }
    }
    __syncthreads();
    const uint32_t result = sh.out_count;
    __syncthreads(); // the next user of `sh` may overwrite out_count at once
    return result;
}

// Sorts records[0..padded) descending; padded is a power of two and the slots
// beyond the live count hold 0 (which sorts last).  Ends with a barrier.
template<int kThreads>
__device__ __noinline__ void block_sort_descending(uint64_t* records, uint32_t padded)
{
    const uint32_t tid = threadIdx.x;
    for (uint32_t size = 2; size <= padded; size <<= 1)
    {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1)
        {
            for (uint32_t i = tid; i < padded; i += kThreads)
            {
                const uint32_t partner = i ^ stride;
                if (partner > i)
                {
                    const bool descending = (i & size) == 0;
                    const uint64_t a = records[i];
                    const uint64_t b = records[partner];
                    if ((a < b) == descending)
                    {
                        records[i] = b;
                        records[partner] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
}

// Position of `mine` among the records of a descending run of 32 (zeros pad
// the tail): the number of entries larger than it.  `run` is the shared-window
// address of the run.
__device__ __forceinline__ uint32_t count_larger_in_run(uint32_t run, uint64_t mine)
{
    uint32_t lo = 0, hi = 32;
#pragma unroll
    for (int step = 0; step < 5; ++step)
    {
        const uint32_t mid = (lo + hi) >> 1;
        if (load_shared_64(run + 8u * mid) > mine)
            lo = mid + 1;
        else
            hi = mid;
    }
    if (lo < 32 && load_shared_64(run + 8u * lo) > mine)
        ++lo;
    return lo;
}

// Sorts records[0..n) (shared memory) descending for n <= kItems * kThreads
// (kItems 1 or 2).  Each warp sorts runs of 32 records in registers with a
// shuffle network; a record's final position is its position in its own run
// plus, for every other run, the number of larger records found by binary
// search — the searches of the different runs are independent, so they are
// unrolled side by side.  Records are unique and 0 pads the tail, so positions
// are unique.  Three barriers, no atomics: the cheapest order for the few
// hundred survivors a slice or a row usually has.  Ends with a barrier.
template<int kThreads, int kItems>
__device__ __forceinline__ void block_rank_sort_items(uint64_t* records, uint32_t n)
{
    constexpr uint32_t kRunsPerItem = kThreads / 32;
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u;
    const uint32_t warp = tid >> 5;
    const uint32_t runs = (n + 31u) >> 5;
    const uint32_t base = shared_address(records);
    uint64_t mine[kItems];
#pragma unroll
    for (int j = 0; j < kItems; ++j)
        mine[j] = (tid + j * kThreads < n) ? load_shared_64(base + 8u * (tid + j * kThreads)) : 0ull;
#pragma unroll
    for (uint32_t size = 2; size <= 32; size <<= 1)
    {
#pragma unroll
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1)
        {
            const bool descending = (lane & size) == 0;
            const bool lower_lane = (lane & stride) == 0;
            const bool take_max = (descending == lower_lane);
#pragma unroll
            for (int j = 0; j < kItems; ++j)
            {
                const uint32_t other_lo = __shfl_xor_sync(kFullMask, static_cast<uint32_t>(mine[j]), stride);
                const uint32_t other_hi = __shfl_xor_sync(kFullMask, static_cast<uint32_t>(mine[j] >> 32), stride);
                const uint64_t other = (static_cast<uint64_t>(other_hi) << 32) | other_lo;
                mine[j] = ((mine[j] > other) == take_max) ? mine[j] : other;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kItems; ++j)
        if (warp + j * kRunsPerItem < runs)
            store_shared_64(base + 8u * (tid + j * kThreads), mine[j]); // run `warp + j * kRunsPerItem`, descending, zeros last
    __syncthreads();
    uint32_t position[kItems];
#pragma unroll
    for (int j = 0; j < kItems; ++j)
    {
        position[j] = lane;
        const uint32_t own = warp + j * kRunsPerItem;
        if (mine[j] != 0ull)
        {
#pragma unroll
            for (uint32_t w = 0; w < kItems * kRunsPerItem; ++w)
                if (w < runs && w != own)
                    position[j] += count_larger_in_run(base + 256u * w, mine[j]);
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kItems; ++j)
        if (mine[j] != 0ull)
            store_shared_64(base + 8u * position[j], mine[j]);
    __syncthreads();
}

template<int kThreads>
__device__ __noinline__ void block_rank_sort_descending(uint64_t* records, uint32_t n)
{
    block_rank_sort_items<kThreads, 1>(records, n);
}

// n <= 2 * kThreads
template<int kThreads>
__device__ __noinline__ void block_rank_sort_descending2(uint64_t* records, uint32_t n)
{
    block_rank_sort_items<kThreads, 2>(records, n);
}

__device__ __forceinline__ uint32_t next_pow2(uint32_t v)
{
    return (v <= 1) ? 1u : (1u << (32 - __clz(static_cast<int>(v - 1))));
}

} // namespace moe
