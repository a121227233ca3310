// Exact full-vocabulary sampler for the rows the streaming kernel hands over:
// rows without Top-K (or with top_k > MOE_SAMPLER_TOPK_FAST_MAX) whose
// numerically live candidate set does not fit in shared memory.
//
// The reference's result for such a row depends on the complete rank order
// (src/engine/session.cpp:80-82) because its softmax normaliser, Top-P
// cumulative, renormaliser and inverse CDF are all left-to-right fp32 sums in
// that order (:92-101,119-134,434-440).  One CTA therefore builds the order of
// all finite logits of the row with a stable least-significant-digit radix
// sort in a per-CTA global scratch slot (L2 resident), and replays the sums over
// it bit-exactly with a block-parallel scan (moe_seqscan.cuh).
//
// CTAs take rows round-robin from the hand-over list; nobody waits on another
// CTA.  The last CTA to finish clears the list for the next call.

#include "moe_common.cuh"
#include "moe_epilogue.cuh"
#include "moe_internal.h"
#include "moe_seqscan.cuh"
#include "moe_seqruns.cuh"

#ifdef MOE_PHASE_TIMERS
// Debug builds only: cycles per phase of the exact kernel, summed over rows.
__device__ unsigned long long g_exact_cycles[16];
extern "C" void moe_debug_exact_cycles(unsigned long long* out, int reset)
{
    cudaMemcpyFromSymbol(out, g_exact_cycles, sizeof(unsigned long long) * 16);
    if (reset)
    {
        unsigned long long zeros[16] = {};
        cudaMemcpyToSymbol(g_exact_cycles, zeros, sizeof(zeros));
    }
}
#define MOE_EXACT_MARK(slot)                                                                              \
    do                                                                                                    \
    {                                                                                                     \
        if (threadIdx.x == 0)                                                                             \
        {                                                                                                 \
            const long long now = clock64();                                                              \
            atomicAdd(&g_exact_cycles[slot], static_cast<unsigned long long>(now - exact_phase_start));   \
            exact_phase_start = now;                                                                      \
        }                                                                                                 \
    } while (0)
#define MOE_EXACT_BEGIN() long long exact_phase_start = clock64()
#else
#define MOE_EXACT_MARK(slot) do {} while (0)
#define MOE_EXACT_BEGIN() do {} while (0)
#endif

namespace moe {

namespace {

constexpr int kExactThreads = 1024;
constexpr int kExactWarps = kExactThreads / 32;
constexpr int kSeqItems = 8; // elements per thread and scan step of the sequential sums

struct ExactShared
{
    SeqShared<1024> seq;
    SeqRunsShared<1024> seq_runs;
    uint32_t run_total;     // value-histogram path: distinct live values of the row
    uint32_t window_total;  // ... and finite logits inside the live window
    uint32_t chosen_warp;   // ... warp whose segment holds the drawn occurrence
    uint32_t chosen_index;
    uint32_t first_fail; // Min-P: first rank whose probability is below the floor
    uint32_t next_entry; // entry of the row queue this CTA took
    uint32_t warp_hist[kExactWarps][256];
    uint32_t digit_total[256];
    uint32_t warp_count[kExactWarps];
    uint32_t warp_or[kExactWarps];
    uint32_t warp_and[kExactWarps];
    uint32_t flag_pos_inf;
    uint32_t total;
    uint32_t finite_total; // finite logits of the row
    uint32_t max_key;      // ordered key of the largest finite logit
    uint32_t min_live_key; // ordered key of the smallest logit compact_live kept
    uint32_t floor_bucket; // coarse bucket below which every logit is numerically dead
    float warp_sum[kExactWarps];
};

// Coarse value buckets of the dead-tail filter: the top 12 bits of the ordered
// key (sign, exponent, three mantissa bits).
constexpr int kCoarseShift = 20;
constexpr uint32_t kCoarseBuckets = 1u << (32 - kCoarseShift);
static_assert(kCoarseBuckets <= kExactWarps * 256u, "the coarse histogram lives in warp_hist");

template<typename T>
__device__ __forceinline__ float load_logit(const T* row, uint32_t index)
{
    return LogitTraits<T>::widen(row, index);
}

// Dead-tail filter.  In rank order a candidate is added to every running sum of
// the reference (session.cpp:92-101,119-134,434-440) after all larger ones, so
// the accumulator it meets is at least their sum; an addend below 2^-25 of the
// accumulator is less than half a unit in its last place and leaves it
// unchanged.  One sweep builds a histogram of the row over coarse value
// buckets; with S(b) = a lower bound of sum(exp(l/T - peak)) over the buckets
// >= b and E(b) = exp(lower edge of b / T - peak), every logit below the lower
// edge of b is dead in all four sums as soon as E(b) <= 2^-27 * 0.9 * S(b) (the factor four
// covers the rounding of the sequential sums and of the normalising
// divisions).  Only the logits at or above the highest such edge are sorted.
// Sets sh.finite_total, sh.max_key, sh.flag_pos_inf and returns the ordered
// key of that edge (0: keep every finite logit).
template<typename T>
__device__ uint32_t dead_tail_floor(const T* row, uint32_t vocab, float temperature, ExactShared& sh)
{
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    uint32_t* const coarse = &sh.warp_hist[0][0];
    for (uint32_t b = tid; b < kCoarseBuckets; b += kExactThreads)
        coarse[b] = 0;
    if (tid == 0)
    {
        sh.flag_pos_inf = 0;
        sh.finite_total = 0;
        sh.max_key = 0;
        sh.floor_bucket = 0;
    }
    __syncthreads();
    uint32_t finite = 0;
    uint32_t max_key = 0;
    bool saw_pos_inf = false;
    for (uint32_t base = 0; base < vocab; base += 4 * kExactThreads)
    {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * kExactThreads + tid;
            v[u] = (i < vocab) ? load_logit(row, i) : __uint_as_float(0x7FC00000u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            saw_pos_inf |= (v[u] == INFINITY);
            if (fabsf(v[u]) < INFINITY)
            {
                const uint32_t key = ordered_key(v[u]);
                atomicAdd(&coarse[key >> kCoarseShift], 1u);
                max_key = max(max_key, key);
                ++finite;
            }
        }
    }
    finite = __reduce_add_sync(kFullMask, finite);
    max_key = __reduce_max_sync(kFullMask, max_key);
    const bool warp_saw_pos_inf = __any_sync(kFullMask, saw_pos_inf);
    if (lane == 0)
    {
        atomicAdd(&sh.finite_total, finite);
        atomicMax(&sh.max_key, max_key);
        if (warp_saw_pos_inf)
            sh.flag_pos_inf = 1;
    }
    __syncthreads();
    if (sh.finite_total == 0 || sh.flag_pos_inf != 0)
        return 0u;
    const float peak = __fdiv_rn(key_to_float(sh.max_key), temperature);
    // thread t owns the four buckets 4t..4t+3 counted from the top
    constexpr int kPerThread = kCoarseBuckets / kExactThreads;
    float edge_exp[kPerThread];
    float mine[kPerThread];
    float running = 0.0f;
#pragma unroll
    for (int j = 0; j < kPerThread; ++j)
    {
        const uint32_t bucket = kCoarseBuckets - 1u - (static_cast<uint32_t>(tid) * kPerThread + j);
        const float edge = key_to_float(bucket << kCoarseShift); // smallest value of the bucket
        const uint32_t count = coarse[bucket];
        // buckets whose edge is not a finite number hold no finite logit; they never become the floor
        edge_exp[j] = (fabsf(edge) < INFINITY) ? expf(fminf(edge / temperature - peak, 0.0f)) : INFINITY;
        if (count != 0)
            running += static_cast<float>(count) * edge_exp[j];
        mine[j] = running;
    }
    // inclusive scan of the per-thread sums, top bucket first
    float scan = running;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1)
    {
        const float other = __shfl_up_sync(kFullMask, scan, offset);
        if (lane >= offset)
            scan += other;
    }
    if (lane == 31)
        sh.warp_sum[warp] = scan;
    __syncthreads();
    float before = scan - running;
    for (int w = 0; w < warp; ++w)
        before += sh.warp_sum[w];
    uint32_t best = 0;
#pragma unroll
    for (int j = 0; j < kPerThread; ++j)
    {
        const uint32_t bucket = kCoarseBuckets - 1u - (static_cast<uint32_t>(tid) * kPerThread + j);
        const float above = before + mine[j]; // lower bound of the sum over the buckets >= this one
        if (edge_exp[j] <= above * (0.9f * 7.450580596923828e-09f)) // 2^-27
            best = max(best, bucket);
    }
    best = __reduce_max_sync(kFullMask, best);
    if (lane == 0 && best != 0)
        atomicMax(&sh.floor_bucket, best);
    __syncthreads();
    const uint32_t floor_key = sh.floor_bucket << kCoarseShift;
    __syncthreads(); // warp_hist is reused by the sort
    return floor_key;
}

// Stable compaction of the finite logits at or above `floor_key` into 64-bit
// sort items (inverted ordered key in the high word, token id in the low word),
// index ascending.  The complement of an item is the candidate record the
// epilogue reads, and ascending items are descending records.  Returns the count.
template<typename T>
__device__ uint32_t compact_live(const T* row, uint32_t vocab, uint32_t floor_key, uint64_t* items, ExactShared& sh)
{
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t segment = ((vocab + 4 * kExactThreads - 1) / (4 * kExactThreads)) * 128u; // per warp, whole 128-logit trips
    const uint32_t begin = min(vocab, warp * segment);
    const uint32_t end = min(vocab, begin + segment);
    const uint32_t least = max(floor_key, kKeyNegInf + 1u);
    uint32_t mine = 0;
    uint32_t lowest = 0xFFFFFFFFu;
    if (tid == 0)
        sh.min_live_key = 0xFFFFFFFFu;
    __syncthreads();
    for (uint32_t base = begin; base < end; base += 128)
    {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * 32 + lane;
            v[u] = (i < end) ? load_logit(row, i) : __uint_as_float(0x7FC00000u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t key = ordered_key(v[u]);
            const bool keep = fabsf(v[u]) < INFINITY && key >= least;
            mine += __popc(__ballot_sync(kFullMask, keep));
            if (keep)
                lowest = min(lowest, key);
        }
    }
    lowest = __reduce_min_sync(kFullMask, lowest);
    if (lane == 0)
    {
        sh.warp_count[warp] = mine;
        atomicMin(&sh.min_live_key, lowest);
    }
    __syncthreads();
    if (warp == 0)
    {
        const uint32_t value = sh.warp_count[lane];
        uint32_t inclusive = value;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1)
        {
            const uint32_t other = __shfl_up_sync(kFullMask, inclusive, offset);
            if (lane >= offset)
                inclusive += other;
        }
        sh.warp_count[lane] = inclusive - value;
        if (lane == 31)
            sh.total = inclusive;
    }
    __syncthreads();
    uint32_t cursor = sh.warp_count[warp];
    for (uint32_t base = begin; base < end; base += 128)
    {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * 32 + lane;
            v[u] = (i < end) ? load_logit(row, i) : __uint_as_float(0x7FC00000u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * 32 + lane;
            const uint32_t key = ordered_key(v[u]);
            const bool keep = fabsf(v[u]) < INFINITY && key >= least;
            const unsigned voters = __ballot_sync(kFullMask, keep);
            if (keep)
            {
                const uint32_t slot = cursor + __popc(voters & ((1u << lane) - 1u));
                items[slot] = (static_cast<uint64_t>(~key) << 32) | i; // ascending sort of this = descending logits
            }
            cursor += __popc(voters);
        }
    }
    __syncthreads();
    return sh.total;
}

// One stable counting-sort pass on an 8-bit digit.  Each warp owns a contiguous
// segment of the input, so input order is preserved inside every digit.
__device__ void radix_pass(const uint64_t* items_in, uint64_t* items_out, uint32_t n, int shift, bool complement_output, ExactShared& sh)
{
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t segment = ((n + 4 * kExactThreads - 1) / (4 * kExactThreads)) * 128u; // per warp, whole 128-key trips
    const uint32_t begin = min(n, warp * segment);
    const uint32_t end = min(n, begin + segment);

    for (int d = lane; d < 256; d += 32)
        sh.warp_hist[warp][d] = 0;
    __syncwarp();
    // four coalesced loads in flight per lane: the scratch lives in L2, and a
    // dependent load per 32 keys would leave the warp waiting most of the time
    for (uint32_t base = begin; base < end; base += 128)
    {
        uint32_t key[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * 32 + lane;
            key[u] = (i < end) ? static_cast<uint32_t>(items_in[i] >> 32) : 0u;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * 32 + lane;
            const bool valid = i < end;
            if (valid)
                atomicAdd(&sh.warp_hist[warp][(key[u] >> shift) & 0xFFu], 1u); // the warp's own counters: only its lanes meet here
        }
    }
    __syncthreads();
    // exclusive offsets: digit-major, then warp order
    if (tid < 256)
    {
        uint32_t running = 0;
        for (int w = 0; w < kExactWarps; ++w)
        {
            const uint32_t value = sh.warp_hist[w][tid];
            sh.warp_hist[w][tid] = running;
            running += value;
        }
        sh.digit_total[tid] = running;
    }
    __syncthreads();
    if (warp == 0)
    {
        uint32_t local[8];
        uint32_t sum = 0;
#pragma unroll
        for (int b = 0; b < 8; ++b)
        {
            local[b] = sh.digit_total[lane * 8 + b];
            sum += local[b];
        }
        uint32_t inclusive = sum;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1)
        {
            const uint32_t other = __shfl_up_sync(kFullMask, inclusive, offset);
            if (lane >= offset)
                inclusive += other;
        }
        uint32_t running = inclusive - sum;
#pragma unroll
        for (int b = 0; b < 8; ++b)
        {
            sh.digit_total[lane * 8 + b] = running;
            running += local[b];
        }
    }
    __syncthreads();
    if (tid < 256)
    {
        const uint32_t digit_base = sh.digit_total[tid];
        for (int w = 0; w < kExactWarps; ++w)
            sh.warp_hist[w][tid] += digit_base;
    }
    __syncthreads();
    for (uint32_t base = begin; base < end; base += 128)
    {
        uint64_t item[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * 32 + lane;
            item[u] = (i < end) ? items_in[i] : 0ull;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * 32 + lane;
            const bool valid = i < end;
            const uint32_t digit = valid ? (static_cast<uint32_t>(item[u] >> (32 + shift)) & 0xFFu) : 0u;
            // lanes with my digit: one vote per bit of the digit (far cheaper here than a match instruction)
            unsigned peers = __ballot_sync(kFullMask, valid);
#pragma unroll
            for (int bit = 0; bit < 8; ++bit)
            {
                const unsigned votes = __ballot_sync(kFullMask, (digit >> bit) & 1u);
                peers &= ((digit >> bit) & 1u) ? votes : ~votes;
            }
            if (valid)
            {
                const uint32_t slot = sh.warp_hist[warp][digit] + __popc(peers & ((1u << lane) - 1u));
                items_out[slot] = complement_output ? ~item[u] : item[u]; // one 8-byte store per item
            }
            __syncwarp();
            if (valid && lane == (__ffs(peers) - 1))
                sh.warp_hist[warp][digit] += __popc(peers);
            __syncwarp();
        }
    }
    __syncthreads();
}

// ---- order by value buckets: one scatter and a look inside each bucket -------------------------
//
// The live logits of an fp32 row are spread over a bounded range of values, so a linear map of the
// value onto kOrderBuckets buckets (bucket 0 = the maximum) leaves a handful of candidates per
// bucket.  One pass counts the buckets, one scatters the items into bucket order (the only
// scattered stores of the method: a byte-digit sort pays them four times), and a last pass puts
// each bucket in order: warps take 128 positions of the scattered list at a time, stage the
// buckets that begin there in shared memory and rank every item inside its own bucket.
// Rows whose values pile up (a bucket above kOrderBucketLimit items) keep the byte-digit sort.
constexpr uint32_t kOrderBuckets = 16384;
constexpr uint32_t kOrderBucketLimit = 128;
constexpr uint32_t kOrderChunk = 128;
constexpr uint32_t kOrderStageItems = kOrderChunk + kOrderBucketLimit; // per warp (plus kOrderStagePad readable words behind)
constexpr uint32_t kOrderStagePad = 4;
constexpr size_t kOrderSharedBytes = sizeof(uint32_t) * kOrderBuckets + sizeof(uint64_t) * kExactWarps * (kOrderStageItems + kOrderStagePad);

struct BucketMap
{
    float top;   // largest live logit
    float scale; // buckets per unit of value
};

// Monotone: a larger logit never gets a larger bucket, equal logits share a bucket.
__device__ __forceinline__ uint32_t order_bucket(uint64_t item, const BucketMap& map)
{
    const float value = key_to_float(~static_cast<uint32_t>(item >> 32));
    const float scaled = __fmul_rn(__fsub_rn(map.top, value), map.scale);
    return min(kOrderBuckets - 1u, __float2uint_rz(scaled));
}

// items_in[0..n): the live items in any order.  On success records_out[0..n) holds the candidate
// records (complemented items) in rank order and true is returned; false: nothing usable was written,
// the caller sorts by digits.  `cursor` and `stage` are the kernel's dynamic shared memory.
__device__ bool order_by_buckets(const uint64_t* items_in, uint64_t* scattered, uint64_t* records_out, uint32_t n, uint32_t max_key, uint32_t min_key,
                                 uint32_t* cursor, uint64_t* stage, ExactShared& sh)
{
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u;
    const uint32_t warp = tid >> 5;
    BucketMap map;
    map.top = key_to_float(max_key);
    const float range = __fsub_rn(map.top, key_to_float(min_key));
    if (!(range > 0.0f) || !(range < INFINITY))
        return false; // one value, or a span fp32 cannot hold
    map.scale = __fdiv_rn(static_cast<float>(kOrderBuckets - 1u), range);
    if (!(map.scale < INFINITY))
        return false;

    for (uint32_t b = tid; b < kOrderBuckets; b += kExactThreads)
        cursor[b] = 0;
    __syncthreads();
    for (uint32_t base = 0; base < n; base += 4u * kExactThreads)
    {
        uint64_t item[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * kExactThreads + tid;
            item[u] = i < n ? items_in[i] : 0ull;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (base + u * kExactThreads + tid < n)
                atomicAdd(&cursor[order_bucket(item[u], map)], 1u);
    }
    __syncthreads();
    // exclusive scan of the counts (consecutive buckets per thread) and the largest bucket
    constexpr uint32_t kPerThread = kOrderBuckets / kExactThreads;
    uint32_t counts[kPerThread];
    uint32_t sum = 0, largest = 0;
#pragma unroll
    for (uint32_t j = 0; j < kPerThread; ++j)
    {
        counts[j] = cursor[tid * kPerThread + j];
        sum += counts[j];
        largest = max(largest, counts[j]);
    }
    uint32_t scan = sum;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1)
    {
        const uint32_t other = __shfl_up_sync(kFullMask, scan, offset);
        if (lane >= static_cast<uint32_t>(offset))
            scan += other;
    }
    largest = __reduce_max_sync(kFullMask, largest);
    if (lane == 31)
        sh.warp_count[warp] = scan;
    if (lane == 0)
        sh.warp_or[warp] = largest;
    __syncthreads();
    uint32_t before = scan - sum;
    for (uint32_t w = 0; w < kExactWarps; ++w)
    {
        if (w < warp)
            before += sh.warp_count[w];
        largest = max(largest, sh.warp_or[w]);
    }
    __syncthreads();
    if (largest > kOrderBucketLimit)
        return false;
#pragma unroll
    for (uint32_t j = 0; j < kPerThread; ++j)
    {
        cursor[tid * kPerThread + j] = before;
        before += counts[j];
    }
    __syncthreads();
    // scatter: the slot comes from the bucket's cursor, which ends at the end of its bucket
    for (uint32_t base = 0; base < n; base += 4u * kExactThreads)
    {
        uint64_t item[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t i = base + u * kExactThreads + tid;
            item[u] = i < n ? items_in[i] : 0ull;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (base + u * kExactThreads + tid < n)
                scattered[atomicAdd(&cursor[order_bucket(item[u], map)], 1u)] = item[u];
    }
    __syncthreads();
    // order inside the buckets
    uint64_t* const mine = stage + static_cast<size_t>(warp) * (kOrderStageItems + kOrderStagePad);
    const uint32_t chunks = (n + kOrderChunk - 1u) / kOrderChunk;
    for (uint32_t chunk = warp; chunk < chunks; chunk += kExactWarps)
    {
        // The window: the chunk's positions and the longest bucket that may reach past them.  The
        // chunk owns the buckets that begin inside its positions; where those begin and end follows
        // from the buckets of the items at the chunk's first position and at the next chunk's.
        const uint32_t window_begin = chunk * kOrderChunk;
        const uint32_t window_count = min(n - window_begin, kOrderStageItems);
        constexpr uint32_t kPerLane = kOrderStageItems / 32u;
        uint64_t held[kPerLane];
#pragma unroll
        for (uint32_t u = 0; u < kPerLane; ++u)
        {
            const uint32_t i = lane + 32u * u;
            held[u] = i < window_count ? scattered[window_begin + i] : ~0ull; // the padding ranks above everything
        }
#pragma unroll
        for (uint32_t u = 0; u < kPerLane; ++u)
            mine[lane + 32u * u] = held[u];
        if (lane < kOrderStagePad)
            mine[kOrderStageItems + lane] = ~0ull;
        __syncwarp();
        // first position the chunk owns: the start of the first bucket that begins at or after window_begin
        const uint32_t head_bucket = order_bucket(mine[0], map);
        const uint32_t head_start = head_bucket == 0u ? 0u : cursor[head_bucket - 1u];
        const uint32_t begin = head_start == window_begin ? window_begin : cursor[head_bucket];
        uint32_t end = n;
        if (window_begin + kOrderChunk < n)
        {
            const uint32_t next_bucket = order_bucket(mine[kOrderChunk], map);
            const uint32_t next_start = next_bucket == 0u ? 0u : cursor[next_bucket - 1u];
            end = next_start == window_begin + kOrderChunk ? next_start : cursor[next_bucket];
        }
#pragma unroll
        for (uint32_t u = 0; u < kPerLane; ++u)
        {
            const uint32_t position = window_begin + lane + 32u * u;
            if (position < begin || position >= end)
                continue;
            const uint64_t item = held[u];
            const uint32_t bucket = order_bucket(item, map);
            const uint32_t bucket_begin = bucket == 0u ? 0u : cursor[bucket - 1u];
            const uint32_t bucket_end = cursor[bucket];
            // what follows a bucket in the window is larger (later buckets, then the padding), so whole
            // trips of four need no guard
            uint32_t rank = 0;
            for (uint32_t j = bucket_begin - window_begin; j < bucket_end - window_begin; j += 4u)
                rank += (mine[j] < item ? 1u : 0u) + (mine[j + 1u] < item ? 1u : 0u) + (mine[j + 2u] < item ? 1u : 0u) + (mine[j + 3u] < item ? 1u : 0u);
            records_out[bucket_begin + rank] = ~item;
        }
        __syncwarp();
    }
    __syncthreads();
    return true;
}

// The arithmetic tail of session.cpp:89-136,429-442 for a complete, sorted
// candidate list of any length, by the whole block: per-candidate exp and
// divisions are spread over the threads, the four running sums are replayed
// bit-exactly by block_sequential_sum.  Same steps, same roundings and same
// outcomes as finish_row_warp (which serves the short lists of the streaming
// kernel); every thread returns the same result.
// `records` holds the first `present` candidates of the rank order; the
// row has `finite_total` finite logits, and those missing from `records` are
// numerically dead (dead_tail_floor).  When the outcome would depend on a
// missing candidate (Min-P prefix or last-candidate fallback reaching past
// `present`), sets needs_full and returns: the caller repeats the row unfiltered.
__device__ RowOutcome finish_row_exact_block(const uint64_t* records, uint32_t present, uint32_t finite_total, float* work, float temperature,
                                             uint32_t top_k, float top_p, float min_p, float uniform, ExactShared& sh, bool& needs_full,
                                             const KeptList& kept_list)
{
    const uint32_t tid = threadIdx.x;
    RowOutcome out{MOE_ROW_OK, -1, 0.0f, 0u, false};
    needs_full = false;
    if (kept_list.count != nullptr && tid == 0)
        *kept_list.count = 0; // stays 0 on every error return
    if (present == 0)
    {
        out.status = MOE_ROW_NO_FINITE_LOGIT;
        return out;
    }
    const uint32_t head_key = record_key(records[0]);
    if (head_key >= kKeyPosInf || head_key <= kKeyNegInf)
    {
        out.status = MOE_ROW_NO_FINITE_LOGIT;
        return out;
    }
    // every candidate is finite (the compaction dropped the rest), so Top-K only shortens the list (session.cpp:86-87)
    const uint32_t listed = (top_k > 0 && top_k < finite_total) ? top_k : finite_total;
    const uint32_t have = min(present, listed); // candidates of the list whose records exist

    MOE_EXACT_BEGIN();
    const float peak = __fdiv_rn(key_to_float(head_key), temperature);
    for (uint32_t i = tid; i < have; i += kExactThreads)
        work[i] = exact_expf(scaled_offset(key_to_float(record_key(records[i])), temperature, peak));
    __syncthreads();
    MOE_EXACT_MARK(8);
    const float total = block_sequential_sum<kExactThreads, kSeqItems>(work, have, kSeqSumOnly, 0.0f, sh.seq).acc;
    MOE_EXACT_MARK(9);
    if (!(total - total == 0.0f) || total <= 0.0f)
    {
        out.status = MOE_ROW_INVALID_DISTRIBUTION;
        return out;
    }
    for (uint32_t i = tid; i < have; i += kExactThreads)
        work[i] = __fdiv_rn(work[i], total);
    if (tid == 0)
        sh.first_fail = have;
    __syncthreads();
    // Min-P: probabilities are non-increasing, so the survivors are a prefix
    uint32_t allowed = listed;
    if (min_p > 0.0f)
    {
        const float floor_probability = __fmul_rn(work[0], min_p);
        uint32_t mine = have;
        for (uint32_t i = tid; i < have; i += kExactThreads)
            if (!(work[i] >= floor_probability))
            {
                mine = i;
                break; // my indices ascend: the first failure is my smallest
            }
        if (mine < have)
            atomicMin(&sh.first_fail, mine);
        __syncthreads();
        const uint32_t first_fail = sh.first_fail;
        __syncthreads();
        if (first_fail < have)
            allowed = first_fail;
        else if (have < listed)
        {
            needs_full = true; // the prefix may go on among the filtered candidates
            return out;
        }
    }
    MOE_EXACT_MARK(10);
    // Top-P: first prefix whose running sum reaches top_p; never reached: the whole list stays
    const SeqResult nucleus = block_sequential_sum<kExactThreads, kSeqItems>(work, min(allowed, have), kSeqReachBound, top_p, sh.seq);
    MOE_EXACT_MARK(11);
    const uint32_t kept = nucleus.stopped ? nucleus.taken : allowed;
    // the renormaliser (session.cpp:130-132) repeats the adds of the Top-P loop over the same prefix from the same zero
    const float kept_total = nucleus.acc;
    if (kept_list.count != nullptr && min(kept, kept_list.stride) > have)
    {
        needs_full = true; // the caller wants candidates that were filtered
        return out;
    }
    if (kept == 1)
    {
        out.token = static_cast<int32_t>(record_index(records[0]));
        out.probability = 1.0f;
        if (kept_list.count != nullptr && tid == 0)
        {
            *kept_list.count = 1;
            if (kept_list.stride > 0)
            {
                if (kept_list.token != nullptr)
                    kept_list.token[0] = out.token;
                if (kept_list.probability != nullptr)
                    kept_list.probability[0] = 1.0f;
            }
        }
        return out;
    }
    out.flags |= MOE_ROW_FLAG_USED_UNIFORM;
    const uint32_t kept_have = min(kept, have);
    for (uint32_t i = tid; i < kept_have; i += kExactThreads)
        work[i] = __fdiv_rn(work[i], kept_total);
    __syncthreads();
    if (kept_list.count != nullptr)
    {
        if (tid == 0)
            *kept_list.count = kept;
        for (uint32_t i = tid; i < min(kept_have, kept_list.stride); i += kExactThreads)
        {
            if (kept_list.token != nullptr)
                kept_list.token[i] = static_cast<int32_t>(record_index(records[i]));
            if (kept_list.probability != nullptr)
                kept_list.probability[i] = work[i];
        }
    }
    MOE_EXACT_MARK(12);
    const SeqResult draw = block_sequential_sum<kExactThreads, kSeqItems>(work, kept_have, kSeqExceedBound, uniform, sh.seq);
    MOE_EXACT_MARK(13);
    uint32_t chosen;
    if (draw.stopped)
        chosen = draw.taken - 1;
    else if (kept <= have)
        chosen = kept - 1; // session.cpp:441-442: the last candidate if the sum never passes the uniform
    else
    {
        needs_full = true; // the last candidate of the list is a filtered one
        return out;
    }
    out.token = static_cast<int32_t>(record_index(records[chosen]));
    out.probability = work[chosen];
    return out;
}

// ---- bf16 rows: a value histogram instead of a sort ---------------------------------
//
// A bf16 row holds at most 65536 distinct logits, a few thousand inside the
// window that can matter, so its rank order is a short list of (value, count)
// runs: candidates of equal value are adjacent, in index order.  The sums are
// replayed over the runs (moe_seqruns.cuh), and the drawn rank (run r, copy j)
// is the j-th lowest index that carries value r, found by one more pass.
// Everything below the window of the row maximum is numerically dead
// (live_window_floor); where the outcome would reach into it, or the caller
// wants per-candidate lists, the sort path takes the row.

constexpr uint32_t kHistogramBins = 40960;        // 160 KiB of dynamic shared memory
constexpr uint32_t kRunsPerThread = 6;            // runs a thread handles in the sums
constexpr uint32_t kMaxRuns = kExactThreads * kRunsPerThread;

// Lowest logit that can still change one of the running sums: exp((v - peak) / T)
// below 2^-26 is absorbed by every accumulator (each starts at the head
// candidate's addend).  0.1 T of slack plus 2^-20 of the peak's magnitude cover
// the roundings of the reference's own v / T - peak / T.
__device__ __forceinline__ float live_window_floor(float peak_logit, float temperature)
{
    return __fsub_rn(__fsub_rn(peak_logit, __fmul_rn(18.2f, temperature)), __fmul_rn(9.5367431640625e-07f, fabsf(peak_logit)));
}

// Calls visit(pattern) for every bf16 logit of the row, in no particular order:
// 16-byte loads (eight logits) while the row is 16-byte aligned, two in flight per thread.
template<typename Visit>
__device__ __forceinline__ void for_each_bf16(const uint16_t* bits, uint32_t vocab, Visit visit)
{
    const uint32_t tid = threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(bits) & 15u) != 0u)
    {
        for (uint32_t i = tid; i < vocab; i += kExactThreads)
            visit(bits[i]);
        return;
    }
    const uint4* vectors = reinterpret_cast<const uint4*>(bits);
    const uint32_t vector_count = vocab / 8u;
    const auto visit_vector = [&](const uint4& v) {
        visit(static_cast<uint16_t>(v.x)); visit(static_cast<uint16_t>(v.x >> 16));
        visit(static_cast<uint16_t>(v.y)); visit(static_cast<uint16_t>(v.y >> 16));
        visit(static_cast<uint16_t>(v.z)); visit(static_cast<uint16_t>(v.z >> 16));
        visit(static_cast<uint16_t>(v.w)); visit(static_cast<uint16_t>(v.w >> 16));
    };
    uint32_t index = tid;
    for (; index + kExactThreads < vector_count; index += 2u * kExactThreads)
    {
        const uint4 first = vectors[index];
        const uint4 second = vectors[index + kExactThreads];
        visit_vector(first);
        visit_vector(second);
    }
    if (index < vector_count)
        visit_vector(vectors[index]);
    for (uint32_t i = vector_count * 8u + tid; i < vocab; i += kExactThreads)
        visit(bits[i]);
}

// Returns false when the row has to go through the sort path; `out` is only valid on true.
__device__ bool exact_row_bf16_runs(const SampleArgs& a, uint32_t row, const moe_row_params& p, uint32_t* hist, uint32_t* scratch, uint32_t scratch_words,
                                    ExactShared& sh, RowOutcome& out)
{
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u;
    const uint32_t warp = tid >> 5;
    const uint16_t* bits = reinterpret_cast<const uint16_t*>(a.logits) + static_cast<size_t>(row) * a.row_stride;
    const uint32_t vocab = a.vocab;
    out = RowOutcome{MOE_ROW_OK, -1, 0.0f, 0u, false};
    if (a.kept_count != nullptr || (a.topk_index != nullptr && p.top_k > 0 && p.top_k <= MOE_SAMPLER_TOPK_FAST_MAX))
        return false; // per-candidate lists need the materialised order
    if (scratch_words < 4u * kMaxRuns)
        return false;

    MOE_EXACT_BEGIN();
    // ---- pass 1: maximum, finite count, +inf --------------------------------------------
    if (tid == 0)
    {
        sh.flag_pos_inf = 0;
        sh.finite_total = 0;
        sh.max_key = 0;
        sh.run_total = 0;
        sh.window_total = 0;
    }
    __syncthreads();
    uint32_t finite = 0, max_key = 0;
    bool saw_pos_inf = false;
    for_each_bf16(bits, vocab, [&](uint16_t pattern) {
        const float v = __uint_as_float(static_cast<uint32_t>(pattern) << 16);
        saw_pos_inf |= (v == INFINITY);
        if (fabsf(v) < INFINITY)
        {
            max_key = max(max_key, ordered_key(v));
            ++finite;
        }
    });
    finite = __reduce_add_sync(kFullMask, finite);
    max_key = __reduce_max_sync(kFullMask, max_key);
    const bool warp_saw_pos_inf = __any_sync(kFullMask, saw_pos_inf);
    if (lane == 0)
    {
        atomicAdd(&sh.finite_total, finite);
        atomicMax(&sh.max_key, max_key);
        if (warp_saw_pos_inf)
            sh.flag_pos_inf = 1;
    }
    __syncthreads();
    const uint32_t finite_total = sh.finite_total;
    MOE_EXACT_MARK(8);
    if (sh.flag_pos_inf != 0 || finite_total == 0)
    {
        out.status = MOE_ROW_NO_FINITE_LOGIT; // session.cpp:84-85,399
        return true;
    }
    const uint32_t top_bin_key = sh.max_key >> 16; // bf16 values: the low half of the ordered key is constant per sign
    const float peak_logit = key_to_float(sh.max_key);
    const float floor_value = live_window_floor(peak_logit, p.temperature);
    // the bin of the floor itself is kept whole: a superset of the live window
    const uint32_t floor_bin_key = (floor_value == floor_value && floor_value > -INFINITY) ? (ordered_key(floor_value) >> 16) : (kKeyNegInf >> 16) + 1u;
    if (floor_bin_key > top_bin_key)
        return false;
    const uint32_t bins = top_bin_key - floor_bin_key + 1u;
    if (bins > kHistogramBins)
        return false;

    // ---- pass 2: histogram over the values of the window, bin 0 = the maximum ------------------
    for (uint32_t b = tid; b < bins; b += kExactThreads)
        hist[b] = 0;
    __syncthreads();
    uint32_t inside = 0;
    for_each_bf16(bits, vocab, [&](uint16_t pattern) {
        const float v = __uint_as_float(static_cast<uint32_t>(pattern) << 16);
        if (fabsf(v) < INFINITY)
        {
            const uint32_t bin_key = ordered_key(v) >> 16;
            if (bin_key >= floor_bin_key)
            {
                atomicAdd(&hist[top_bin_key - bin_key], 1u);
                ++inside;
            }
        }
    });
    inside = __reduce_add_sync(kFullMask, inside);
    if (lane == 0 && inside != 0)
        atomicAdd(&sh.window_total, inside);
    __syncthreads();
    const uint32_t window_total = sh.window_total;
    MOE_EXACT_MARK(9);

    // ---- runs: the non-empty bins in rank order, with the number of candidates before each -------
    // built in the global scratch slot, then moved into shared memory
    float* run_value = reinterpret_cast<float*>(scratch);       // addend of the run (numerator, probability, ...)
    uint32_t* run_count = scratch + kMaxRuns;
    uint32_t* run_cum = scratch + 2u * kMaxRuns;
    uint32_t* run_key = scratch + 3u * kMaxRuns;                 // ordered key of the run's logit
    const uint32_t bins_per_thread = (bins + kExactThreads - 1u) / kExactThreads;
    const uint32_t my_first_bin = min(bins, tid * bins_per_thread);
    const uint32_t my_last_bin = min(bins, my_first_bin + bins_per_thread);
    uint32_t my_runs = 0, my_elements = 0;
    for (uint32_t b = my_first_bin; b < my_last_bin; ++b)
    {
        const uint32_t c = hist[b];
        my_runs += c != 0 ? 1u : 0u;
        my_elements += c;
    }
    // block-wide exclusive scan of (runs, elements)
    uint32_t scan_runs = my_runs, scan_elements = my_elements;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1)
    {
        const uint32_t r = __shfl_up_sync(kFullMask, scan_runs, offset);
        const uint32_t e = __shfl_up_sync(kFullMask, scan_elements, offset);
        if (lane >= static_cast<uint32_t>(offset))
        {
            scan_runs += r;
            scan_elements += e;
        }
    }
    if (lane == 31)
    {
        sh.warp_count[warp] = scan_runs;
        sh.warp_or[warp] = scan_elements;
    }
    __syncthreads();
    uint32_t runs_before = scan_runs - my_runs, elements_before = scan_elements - my_elements;
    for (uint32_t w = 0; w < warp; ++w)
    {
        runs_before += sh.warp_count[w];
        elements_before += sh.warp_or[w];
    }
    if (tid == kExactThreads - 1)
        sh.run_total = runs_before + my_runs;
    __syncthreads();
    const uint32_t runs = sh.run_total;
    if (runs > kMaxRuns)
        return false;
    for (uint32_t b = my_first_bin; b < my_last_bin; ++b)
    {
        const uint32_t c = hist[b];
        if (c != 0)
        {
            run_count[runs_before] = c;
            run_cum[runs_before] = elements_before;
            // ordered key of the bf16 value of this bin: its low half is all zeros for a
            // non-negative value and all ones for a negative one (the complemented zero bits)
            const uint32_t bin_key = top_bin_key - b;
            run_key[runs_before] = (bin_key << 16) | ((bin_key & 0x8000u) ? 0u : 0xFFFFu);
            ++runs_before;
            elements_before += c;
        }
    }
    __syncthreads();
    // The histogram has served its purpose: its shared memory now holds the run arrays, which the
    // sums below walk many times (4 * runs <= 4 * kMaxRuns words fit the kHistogramBins words).
    static_assert(5u * kMaxRuns <= kHistogramBins, "the run arrays and the replay guide reuse the histogram's shared memory");
    float* const run_guide = reinterpret_cast<float*>(hist + 4u * kMaxRuns); // approximate prefix sums of the numerators
    {
        float* shared_value = reinterpret_cast<float*>(hist);
        uint32_t* shared_count = hist + kMaxRuns;
        uint32_t* shared_cum = hist + 2u * kMaxRuns;
        uint32_t* shared_key = hist + 3u * kMaxRuns;
        for (uint32_t r = tid; r < runs; r += kExactThreads)
        {
            shared_count[r] = run_count[r];
            shared_cum[r] = run_cum[r];
            shared_key[r] = run_key[r];
        }
        __syncthreads();
        run_value = shared_value;
        run_count = shared_count;
        run_cum = shared_cum;
        run_key = shared_key;
    }

    MOE_EXACT_MARK(10);
    // ---- the arithmetic of session.cpp:89-136,429-442 over the runs --------------------------
    // Top-K (only top_k > MOE_SAMPLER_TOPK_FAST_MAX reaches this kernel) shortens the list
    const uint32_t listed = (p.top_k > 0 && p.top_k < finite_total) ? p.top_k : finite_total;
    const uint32_t have = min(window_total, listed); // candidates whose runs exist
    const float peak = __fdiv_rn(peak_logit, p.temperature);
    for (uint32_t r = tid; r < runs; r += kExactThreads)
        run_value[r] = exact_expf(scaled_offset(key_to_float(run_key[r]), p.temperature, peak));
    __syncthreads();
    block_runs_prefix_guide<kExactThreads, kRunsPerThread>(run_value, run_count, runs, run_guide, sh.warp_sum);
    const SeqRunsResult normaliser = block_sequential_sum_runs<kExactThreads, kRunsPerThread>(run_value, run_count, run_cum, runs, have, kSeqSumOnly, 0.0f, sh.seq_runs,
                                                                                              run_guide, 1.0f);
    if (normaliser.unsupported)
        return false;
    MOE_EXACT_MARK(11);
    const float total = normaliser.acc;
    if (!(total - total == 0.0f) || total <= 0.0f)
    {
        out.status = MOE_ROW_INVALID_DISTRIBUTION; // session.cpp:102-103
        return true;
    }
    for (uint32_t r = tid; r < runs; r += kExactThreads)
        run_value[r] = __fdiv_rn(run_value[r], total);
    if (tid == 0)
        sh.first_fail = runs;
    __syncthreads();
    // Min-P: probabilities do not increase, so the survivors are a prefix of the runs
    uint32_t allowed = listed;
    if (p.min_p > 0.0f)
    {
        const float floor_probability = __fmul_rn(run_value[0], p.min_p);
        uint32_t mine = runs;
        for (uint32_t r = tid; r < runs; r += kExactThreads)
            if (!(run_value[r] >= floor_probability))
            {
                mine = r;
                break;
            }
        if (mine < runs)
            atomicMin(&sh.first_fail, mine);
        __syncthreads();
        const uint32_t first_fail = sh.first_fail;
        __syncthreads();
        if (first_fail < runs)
            allowed = min(allowed, run_cum[first_fail]);
        else if (have < listed)
            return false; // the prefix may go on below the window
    }
    // Top-P: first prefix whose running sum reaches top_p; never reached: the whole list stays
    const SeqRunsResult nucleus = block_sequential_sum_runs<kExactThreads, kRunsPerThread>(run_value, run_count, run_cum, runs, min(allowed, have), kSeqReachBound, p.top_p, sh.seq_runs,
                                                                                           run_guide, 1.0f / total);
    if (nucleus.unsupported)
        return false;
    MOE_EXACT_MARK(12);
    const uint32_t kept = nucleus.stopped ? nucleus.taken : allowed;
    // the renormaliser (session.cpp:130-132) repeats the adds of the Top-P loop over the same prefix from the same zero
    const float kept_total = nucleus.acc;
    uint32_t chosen_run = 0;
    uint32_t occurrence = 0; // 0-based among the indices carrying the chosen value
    if (kept == 1)
    {
        // session.cpp:429-430: no uniform drawn; the head candidate is the lowest index of the maximum
        out.probability = 1.0f;
    }
    else
    {
        out.flags |= MOE_ROW_FLAG_USED_UNIFORM;
        const uint32_t kept_have = min(kept, have);
        for (uint32_t r = tid; r < runs; r += kExactThreads)
            run_value[r] = __fdiv_rn(run_value[r], kept_total);
        __syncthreads();
        const float uniform = philox_uniform(p.seed, p.row_id, p.step + a.step_offset);
        const SeqRunsResult draw = block_sequential_sum_runs<kExactThreads, kRunsPerThread>(run_value, run_count, run_cum, runs, kept_have, kSeqExceedBound, uniform, sh.seq_runs,
                                                                                            run_guide, 1.0f / (total * kept_total));
        if (draw.unsupported)
            return false;
        uint32_t chosen_rank;
        if (draw.stopped)
            chosen_rank = draw.taken - 1u;
        else if (kept <= have)
            chosen_rank = kept - 1u; // session.cpp:441-442: the last candidate if the sum never passes the uniform
        else
            return false; // the last candidate of the list lies below the window
        // run of that rank: the last run that starts at or before it
        if (tid == 0)
            sh.first_fail = 0;
        __syncthreads();
        {
            uint32_t mine = 0;
            for (uint32_t r = tid; r < runs; r += kExactThreads)
                if (run_cum[r] <= chosen_rank)
                    mine = max(mine, r);
            mine = __reduce_max_sync(kFullMask, mine);
            if (lane == 0)
                atomicMax(&sh.first_fail, mine);
        }
        __syncthreads();
        chosen_run = sh.first_fail;
        occurrence = chosen_rank - run_cum[chosen_run];
        out.probability = run_value[chosen_run];
    }
    const float chosen_value = key_to_float(run_key[chosen_run]);
    const uint16_t wanted = static_cast<uint16_t>(__float_as_uint(chosen_value) >> 16);
    __syncthreads();
    MOE_EXACT_MARK(13);

    // ---- the occurrence-th lowest index that carries the chosen value ------------------------
    // Each warp owns a contiguous part of the row (whole 16-byte vectors) and reads it with
    // consecutive lanes on consecutive vectors, so "lowest" is a prefix count over warps, then
    // over the trips of one warp, then over its lanes.
    const bool aligned = (reinterpret_cast<uintptr_t>(bits) & 15u) == 0u;
    const bool wanted_is_zero = (wanted & 0x7FFFu) == 0u; // +0 and -0 are one value
    const uint32_t wanted_pair = static_cast<uint32_t>(wanted) | (static_cast<uint32_t>(wanted) << 16);
    const auto matches = [&](uint16_t pattern) -> bool { return wanted_is_zero ? (pattern & 0x7FFFu) == 0u : pattern == wanted; };
    // bits 2i, 2i+1 of the result = the two logits of word i carry the value
    const auto pair_mask = [&](uint32_t word) -> uint32_t {
        const uint32_t differs = wanted_is_zero ? (word & 0x7FFF7FFFu) : (word ^ wanted_pair);
        return ((differs & 0xFFFFu) == 0u ? 1u : 0u) | ((differs >> 16) == 0u ? 2u : 0u);
    };
    // bit i of the mask = the i-th logit of the vector carries the value
    const auto vector_mask = [&](const uint4& v) -> uint32_t {
        return pair_mask(v.x) | (pair_mask(v.y) << 2) | (pair_mask(v.z) << 4) | (pair_mask(v.w) << 6);
    };
    // mask of the eight logits that start at `at` (a multiple of 8 inside the warp's part), by vector or one by one
    const auto mask_at = [&](uint32_t at, uint32_t end) -> uint32_t {
        if (at >= end)
            return 0u;
        if (aligned && at + 8u <= end)
            return vector_mask(*reinterpret_cast<const uint4*>(bits + at));
        uint32_t mask = 0;
        for (uint32_t j = 0; j < 8u && at + j < end; ++j)
            mask |= matches(bits[at + j]) ? (1u << j) : 0u;
        return mask;
    };
    const uint32_t part = ((vocab + kExactWarps - 1u) / kExactWarps + 255u) & ~255u; // whole trips of 32 vectors
    const uint32_t begin = min(vocab, warp * part);
    const uint32_t end = min(vocab, begin + part);
    const uint32_t trips = (end - begin + 255u) / 256u;
    // lane g keeps the count of trip group g, so that the second look goes straight to the right trips
    const uint32_t trips_per_group = max(1u, (part / 256u + 31u) / 32u);
    uint32_t in_part = 0, group_total = 0;
    for (uint32_t trip = 0; trip < trips; trip += 4u)
    {
        uint32_t mask[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            mask[u] = trip + u < trips ? mask_at(begin + (trip + u) * 256u + lane * 8u, end) : 0u;
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            const uint32_t total = __reduce_add_sync(kFullMask, __popc(mask[u]));
            in_part += total;
            if (lane == (trip + u) / trips_per_group)
                group_total += total;
        }
    }
    if (lane == 0)
        sh.warp_count[warp] = in_part;
    if (tid == 0)
        sh.chosen_index = 0xFFFFFFFFu;
    __syncthreads();
    uint32_t before = 0;
    for (uint32_t w = 0; w < warp; ++w)
        before += sh.warp_count[w];
    if (occurrence >= before && occurrence < before + in_part)
    {
        // this warp's part holds it: the group of trips first, then the trip, then the lane
        uint32_t inclusive = group_total;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1)
        {
            const uint32_t other = __shfl_up_sync(kFullMask, inclusive, offset);
            if (lane >= static_cast<uint32_t>(offset))
                inclusive += other;
        }
        const unsigned reached = __ballot_sync(kFullMask, occurrence < before + inclusive);
        const uint32_t group = static_cast<uint32_t>(__ffs(reached)) - 1u; // not empty: the last lane holds in_part
        uint32_t seen = before + __shfl_sync(kFullMask, inclusive - group_total, group);
        const uint32_t last_trip = min(trips, (group + 1u) * trips_per_group);
        for (uint32_t trip = group * trips_per_group; trip < last_trip; ++trip)
        {
            const uint32_t at = begin + trip * 256u + lane * 8u;
            uint32_t mask = mask_at(at, end);
            const uint32_t here = __popc(mask);
            uint32_t scan = here;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1)
            {
                const uint32_t other = __shfl_up_sync(kFullMask, scan, offset);
                if (lane >= static_cast<uint32_t>(offset))
                    scan += other;
            }
            const uint32_t mine_first = seen + scan - here;
            if (occurrence >= mine_first && occurrence < mine_first + here)
            {
                for (uint32_t skip = occurrence - mine_first; skip > 0; --skip)
                    mask &= mask - 1u; // drop the lowest set bits
                sh.chosen_index = at + static_cast<uint32_t>(__ffs(mask) - 1);
            }
            seen += __shfl_sync(kFullMask, scan, 31);
            if (seen > occurrence)
                break;
        }
    }
    __syncthreads();
    out.token = static_cast<int32_t>(sh.chosen_index);
    __syncthreads();
    MOE_EXACT_MARK(0);
    return out.token >= 0;
}

template<typename T>
__device__ void exact_row(const SampleArgs& a, uint32_t row, uint32_t* slot_keys, uint32_t* slot_index, uint32_t slot_stride, ExactShared& sh)
{
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const moe_row_params p = a.params[row];
    const T* row_pointer = static_cast<const T*>(a.logits) + static_cast<size_t>(row) * a.row_stride;

    // the slot holds two buffers of slot_stride 64-bit items; the sort ping-pongs between them
    uint64_t* items[2] = {reinterpret_cast<uint64_t*>(slot_keys), reinterpret_cast<uint64_t*>(slot_keys) + slot_stride};
    (void)slot_index;

    MOE_EXACT_BEGIN();
    // rows that list their Top-K ids need every rank up to top_k: no filter for them
    const bool lists = a.topk_index != nullptr && p.top_k > 0 && p.top_k <= MOE_SAMPLER_TOPK_FAST_MAX;
    RowOutcome out{MOE_ROW_OK, -1, 0.0f, 0u, false};
    uint64_t* records = items[0];
    uint32_t n = 0;
    bool handled = false;
    if constexpr (sizeof(T) == 2)
    {
        extern __shared__ __align__(16) uint32_t value_histogram[];
        handled = exact_row_bf16_runs(a, row, p, value_histogram, slot_keys, 4u * slot_stride, sh, out);
        __syncthreads();
        if (handled && a.kept_count != nullptr && tid == 0)
            a.kept_count[row] = 0; // unreachable today (lists go through the sort path); kept for a consistent contract
        MOE_EXACT_MARK(6);
    }
    uint32_t floor_key = 0;
    bool has_pos_inf = false;
    uint32_t finite_total = 0;
    if (!handled)
    {
        floor_key = dead_tail_floor<T>(row_pointer, a.vocab, p.temperature, sh);
        has_pos_inf = sh.flag_pos_inf != 0;
        finite_total = sh.finite_total;
        if (lists)
            floor_key = 0;
        MOE_EXACT_MARK(4);
    }

    if (handled)
    {
        // finished by the value-histogram path
    }
    else if (has_pos_inf || finite_total == 0)
    {
        out.status = MOE_ROW_NO_FINITE_LOGIT;
        if (a.kept_count != nullptr && tid == 0)
            a.kept_count[row] = 0;
    }
    else
    {
        for (int attempt = 0; attempt < 2; ++attempt)
        {
            n = compact_live<T>(row_pointer, a.vocab, floor_key, items[0], sh);
            MOE_EXACT_MARK(0);
            int source = 0;
            bool complemented = false;
            bool ordered = false;
            if constexpr (sizeof(T) == 4)
            {
                if (n > 1)
                {
                    extern __shared__ __align__(16) uint32_t order_words[];
                    ordered = order_by_buckets(items[0], items[1], items[0], n, sh.max_key, sh.min_live_key, order_words,
                                               reinterpret_cast<uint64_t*>(order_words + kOrderBuckets), sh);
                    complemented = ordered;
                }
            }
            if (n > 1 && !ordered)
            {
                // A digit needs no pass when it is the same function of the higher digits
                // for every key.  Keys (high words) are ~ordered_key(v): their low bytes are the
                // magnitude bytes of v, complemented or not by the sign alone, so a byte
                // on which all magnitudes agree (bf16 logits: the two low bytes) can be
                // skipped.  (x ^ (x >> 31 ? 0 : ~0)) & 0x7FFFFFFF recovers the magnitude.
                uint32_t any_bits = 0;
                uint32_t all_bits = 0xFFFFFFFFu;
                for (uint32_t i = tid; i < n; i += kExactThreads)
                {
                    const uint32_t key = static_cast<uint32_t>(items[0][i] >> 32);
                    const uint32_t magnitude = ((key & 0x80000000u) ? key : ~key) & 0x7FFFFFFFu;
                    const uint32_t probe = magnitude | (key & 0x80000000u);
                    any_bits |= probe;
                    all_bits &= probe;
                }
                any_bits = __reduce_or_sync(kFullMask, any_bits);
                all_bits = __reduce_and_sync(kFullMask, all_bits);
                if (lane == 0)
                {
                    sh.warp_or[warp] = any_bits;
                    sh.warp_and[warp] = all_bits;
                }
                __syncthreads();
                any_bits = 0;
                all_bits = 0xFFFFFFFFu;
                for (int w = 0; w < kExactWarps; ++w)
                {
                    any_bits |= sh.warp_or[w];
                    all_bits &= sh.warp_and[w];
                }
                const uint32_t varying = any_bits ^ all_bits;
                __syncthreads();
                // complementing a sorted item gives the candidate record (ordered key,
                // 0xFFFFFFFF - id); the last pass stores the complement directly
                int last_shift = -1;
                for (int shift = 0; shift < 32; shift += 8)
                    if (((varying >> shift) & 0xFFu) != 0)
                        last_shift = shift;
                for (int shift = 0; shift < 32; shift += 8)
                {
                    if (((varying >> shift) & 0xFFu) == 0)
                        continue;
                    radix_pass(items[source], items[1 - source], n, shift, shift == last_shift, sh);
                    source = 1 - source;
                    complemented = shift == last_shift;
                }
            }
            MOE_EXACT_MARK(1);
            // the other buffer is free and serves the epilogue's floats
            records = items[source];
            float* work = reinterpret_cast<float*>(items[1 - source]);
            if (!complemented)
            {
                for (uint32_t i = tid; i < n; i += kExactThreads)
                    records[i] = ~records[i];
                __syncthreads();
            }
            MOE_EXACT_MARK(2);

            const float uniform = philox_uniform(p.seed, p.row_id, p.step + a.step_offset);
            bool needs_full = false;
            out = finish_row_exact_block(records, n, finite_total, work, p.temperature, p.top_k, p.top_p, p.min_p, uniform, sh, needs_full,
                                         kept_list_of_row(a.kept_token, a.kept_probability, a.kept_count, a.kept_stride, row));
            MOE_EXACT_MARK(3);
            if (!needs_full || floor_key == 0)
                break;
            floor_key = 0; // the outcome hangs on a filtered candidate: once more with every finite logit
            __syncthreads();
        }
    }

    if (a.topk_index != nullptr)
    {
        // same contract as the streaming kernel: the rank-ordered ids of a Top-K row, -1 elsewhere
        const bool shown = lists && out.status != MOE_ROW_NO_FINITE_LOGIT && p.temperature != 0.0f;
        const uint32_t listed = shown ? min(n, p.top_k) : 0u;
        for (uint32_t i = tid; i < a.topk_stride; i += kExactThreads)
            a.topk_index[static_cast<size_t>(row) * a.topk_stride + i] = (i < listed) ? static_cast<int32_t>(record_index(records[i])) : -1;
    }

    if (tid == 0)
    {
        if (out.status == MOE_ROW_OK && is_stop_token(a.stop_offsets, a.stop_tokens, row, out.token))
            out.flags |= MOE_ROW_FLAG_STOP_TOKEN;
        a.token_id[row] = out.token;
        a.probability[row] = out.probability;
        if (a.row_flags != nullptr)
            a.row_flags[row] = out.flags;
        if (a.row_status != nullptr)
            a.row_status[row] = out.status;
    }
    __syncthreads();
#ifdef MOE_PHASE_TIMERS
    if (threadIdx.x == 0)
    {
        atomicAdd(&g_exact_cycles[7], 1ull);
        atomicAdd(&g_exact_cycles[5], static_cast<unsigned long long>(n));
    }
#endif
}

template<typename T>
__global__ void __launch_bounds__(kExactThreads, 1) sample_exact_kernel(const SampleArgs a, Workspace ws)
{
    __shared__ ExactShared sh;
    const uint32_t pending = *ws.exact_count;
    const uint32_t slot_stride = (ws.max_vocab + 3u) & ~3u;
    uint32_t* slot_keys = ws.sort_keys + static_cast<size_t>(blockIdx.x) * 4u * slot_stride;
    // rows cost from a few to several hundred microseconds: a CTA takes the next one when it is free
    for (;;)
    {
        if (threadIdx.x == 0)
            sh.next_entry = atomicAdd(ws.exact_next, 1u);
        __syncthreads();
        const uint32_t entry = sh.next_entry;
        __syncthreads();
        if (entry >= pending)
            break;
        exact_row<T>(a, ws.exact_rows[entry], slot_keys, nullptr, slot_stride, sh);
    }
    __syncthreads();
    if (threadIdx.x == 0)
    {
        __threadfence();
        if (atomicAdd(ws.exact_done, 1u) == gridDim.x - 1)
        {
            *ws.exact_count = 0; // every CTA has read it: ready for the next call
            *ws.exact_done = 0;
            *ws.exact_next = 0;
            __threadfence();
        }
    }
}

} // namespace

cudaError_t launch_sample_exact(const SampleArgs& args, const Workspace& ws, cudaStream_t stream)
{
    if (args.rows == 0 || ws.slots == 0)
        return cudaSuccess;
    const uint32_t grid = ws.slots < args.rows ? ws.slots : args.rows;
    if (args.dtype == MOE_DTYPE_F32)
    {
        static SharedOptIn opt_in;
        if (cudaError_t status = opt_in_shared(opt_in, sample_exact_kernel<float>, kOrderSharedBytes))
            return status;
        sample_exact_kernel<float><<<grid, kExactThreads, kOrderSharedBytes, stream>>>(args, ws);
    }
    else
    {
        // the value histogram of the bf16 path lives in dynamic shared memory
        const size_t shared_bytes = sizeof(uint32_t) * kHistogramBins;
        static SharedOptIn opt_in;
        if (cudaError_t status = opt_in_shared(opt_in, sample_exact_kernel<__nv_bfloat16>, shared_bytes))
            return status;
        sample_exact_kernel<__nv_bfloat16><<<grid, kExactThreads, shared_bytes, stream>>>(args, ws);
    }
    return cudaGetLastError();
}

} // namespace moe
