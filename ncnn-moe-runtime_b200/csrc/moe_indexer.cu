// Stable Top-K over rows of scores: the latent-attention indexer's choice of
// compressed history entries (src/kernels/cpu_latent_attention.cpp:377-425 of
// the reference: std::partial_sort of {index, score} pairs with
// scored_index_precedes, :257-262 — score descending, index ascending on equal
// scores — and the first index_top_k indices in that order).
//
// One CTA per row.  The k-th largest key is found by a radix select over the
// 32-bit order-preserving keys of the scores (four 8-bit digits from the top,
// one pass over the row each; the row stays in L2), the entries above it and
// the lowest-index entries equal to it are compacted into shared memory as
// (key, index) records — the record and ordering primitive of the sampler —
// and sorted there.  Scores are read k-independently: 4 + 2 passes of
// count * 4 bytes per row.

#include "moe_common.cuh"
#include "moe_internal.h"
#include "moe_select.cuh"

namespace moe {

namespace {

constexpr int kIndexThreads = 1024;
constexpr int kIndexWarps = kIndexThreads / 32;

struct IndexerShared
{
    uint32_t hist[256];
    uint32_t warp_equal[kIndexWarps];
    uint32_t digit;
    uint32_t above;
    uint32_t taken;
};

// NaN scores make the reference's comparator inconsistent; here they rank last.
__device__ __forceinline__ uint32_t score_key(float value)
{
    return (value == value) ? ordered_key(value) : 0u;
}

__global__ void __launch_bounds__(kIndexThreads) indexer_topk_kernel(const float* scores, uint32_t count, size_t row_stride, uint32_t top_k,
                                                                     uint32_t* out_index, float* out_score)
{
    extern __shared__ __align__(16) unsigned char shared_raw[];
    IndexerShared& sh = *reinterpret_cast<IndexerShared*>(shared_raw);
    uint64_t* records = reinterpret_cast<uint64_t*>(shared_raw + ((sizeof(IndexerShared) + 15u) & ~size_t(15)));
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u;
    const uint32_t warp = tid >> 5;
    const float* row = scores + static_cast<size_t>(blockIdx.x) * row_stride;
    const uint32_t selected = min(top_k, count);
    if (selected == 0)
    {
        for (uint32_t i = tid; i < top_k; i += kIndexThreads)
        {
            out_index[static_cast<size_t>(blockIdx.x) * top_k + i] = 0xFFFFFFFFu;
            if (out_score != nullptr)
                out_score[static_cast<size_t>(blockIdx.x) * top_k + i] = 0.0f;
        }
        return;
    }

    // ---- the selected-th largest key, digit by digit -----------------------------------
    uint32_t prefix = 0;      // digits decided so far (high bits)
    uint32_t prefix_mask = 0;
    uint32_t remaining = selected; // rank still looked for among the keys that match the prefix
    for (int shift = 24; shift >= 0; shift -= 8)
    {
        if (tid < 256)
            sh.hist[tid] = 0;
        __syncthreads();
        for (uint32_t base = 0; base < count; base += kIndexThreads)
        {
            const uint32_t i = base + tid;
            const uint32_t key = i < count ? score_key(row[i]) : 0u;
            const bool match = i < count && (key & prefix_mask) == prefix;
            const uint32_t digit = match ? ((key >> shift) & 0xFFu) : 0xFFFFFFFFu;
            // one shared atomic per distinct digit of the warp
            const unsigned peers = __match_any_sync(kFullMask, digit);
            if (match && lane == static_cast<uint32_t>(__ffs(peers) - 1))
                atomicAdd(&sh.hist[digit], static_cast<uint32_t>(__popc(peers)));
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
            if (static_cast<int>(lane) == owner)
            {
                uint32_t cumulative = suffix - lane_total;
#pragma unroll
                for (int b = 7; b >= 0; --b)
                {
                    if (cumulative + bins[b] >= remaining)
                    {
                        sh.digit = lane * 8 + b;
                        sh.above = cumulative;
                        break;
                    }
                    cumulative += bins[b];
                }
            }
        }
        __syncthreads();
        prefix |= sh.digit << shift;
        prefix_mask |= 0xFFu << shift;
        remaining -= sh.above;
        __syncthreads();
    }
    const uint32_t threshold = prefix;   // the selected-th largest key
    const uint32_t equal_wanted = remaining; // entries equal to it that belong to the selection: the lowest indices

    // ---- compaction: everything above the threshold, and the first `equal_wanted` equal to it ----
    // each warp owns a contiguous run of the row, so that "first" means lowest index
    const uint32_t segment = ((count + kIndexWarps * 32u - 1u) / (kIndexWarps * 32u)) * 32u;
    const uint32_t begin = min(count, warp * segment);
    const uint32_t end = min(count, begin + segment);
    uint32_t equal_here = 0;
    for (uint32_t base = begin; base < end; base += 32)
    {
        const uint32_t i = base + lane;
        const bool equal = i < end && score_key(row[i]) == threshold;
        equal_here += __popc(__ballot_sync(kFullMask, equal));
    }
    if (lane == 0)
        sh.warp_equal[warp] = equal_here;
    if (tid == 0)
        sh.taken = 0;
    __syncthreads();
    uint32_t equal_before = 0; // entries equal to the threshold in the warps before this one
    for (uint32_t w = 0; w < warp; ++w)
        equal_before += sh.warp_equal[w];
    for (uint32_t base = begin; base < end; base += 32)
    {
        const uint32_t i = base + lane;
        const uint32_t key = i < end ? score_key(row[i]) : 0u;
        const bool above = i < end && key > threshold;
        const bool equal = i < end && key == threshold;
        const unsigned equal_votes = __ballot_sync(kFullMask, equal);
        const bool take = above || (equal && equal_before + __popc(equal_votes & ((1u << lane) - 1u)) < equal_wanted);
        const unsigned takers = __ballot_sync(kFullMask, take);
        uint32_t slot = 0;
        if (lane == 0 && takers != 0u)
            slot = atomicAdd(&sh.taken, static_cast<uint32_t>(__popc(takers)));
        slot = __shfl_sync(kFullMask, slot, 0) + __popc(takers & ((1u << lane) - 1u));
        if (take)
            records[slot] = make_record(key, i); // the order of arrival does not matter: the sort below decides
        equal_before += __popc(equal_votes);
    }
    __syncthreads();

    // ---- rank order of the selection --------------------------------------------------
    const uint32_t padded = next_pow2(selected);
    for (uint32_t i = selected + tid; i < padded; i += kIndexThreads)
        records[i] = 0ull;
    __syncthreads();
    block_sort_descending<kIndexThreads>(records, padded);
    for (uint32_t i = tid; i < top_k; i += kIndexThreads)
    {
        const bool filled = i < selected;
        const uint32_t index = filled ? record_index(records[i]) : 0xFFFFFFFFu;
        out_index[static_cast<size_t>(blockIdx.x) * top_k + i] = index;
        if (out_score != nullptr)
            out_score[static_cast<size_t>(blockIdx.x) * top_k + i] = filled ? row[index] : 0.0f;
    }
}

} // namespace

cudaError_t launch_indexer_topk(const float* scores, uint32_t rows, uint32_t count, size_t row_stride, uint32_t top_k, uint32_t* out_index,
                                float* out_score, cudaStream_t stream)
{
    if (rows == 0 || top_k == 0)
        return cudaSuccess;
    const uint32_t selected = top_k < count ? top_k : count;
    uint32_t padded = 1;
    while (padded < selected)
        padded <<= 1;
    const size_t shared_bytes = ((sizeof(IndexerShared) + 15u) & ~size_t(15)) + sizeof(uint64_t) * padded;
    static SharedOptIn opt_in;
    if (shared_bytes > 48u * 1024u)
    {
        if (cudaError_t status = opt_in_shared(opt_in, indexer_topk_kernel, shared_bytes))
            return status;
    }
    indexer_topk_kernel<<<rows, kIndexThreads, shared_bytes, stream>>>(scores, count, row_stride, top_k, out_index, out_score);
    return cudaGetLastError();
}

} // namespace moe
