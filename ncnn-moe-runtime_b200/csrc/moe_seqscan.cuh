// Block-parallel, bit-exact replay of a left-to-right fp32 accumulation
//     acc = 0; for i in 0..n: acc = acc + x[i]      (round to nearest even each step)
// over a non-increasing, non-negative sequence — the shape of all four sums of
// the reference sampler (src/engine/session.cpp:92-101,119-134,434-440).
//
// While the accumulator stays inside one binade [2^b, 2^(b+1)) it is an
// integer multiple A of u = 2^(b-23), and adding x moves A by
//     q + r,   q = floor(x / u),   r = 0 / 1 by the fraction of x / u
//     (below 1/2: 0, above: 1, exactly 1/2: whichever makes A + q + r even).
// Only the tie case looks at the accumulator, and only at its parity, so an
// element is a pair of integer steps (one per parity of A) and two elements
// compose into another such pair: an associative operator, hence a parallel
// prefix scan.  Every thread then knows the exact accumulator after each of
// its elements.  The first element whose step would carry A to 2^24 ends the
// binade; it is added with a real fp32 add and the scan restarts behind it.
// x <= acc always holds here, so a step never exceeds 2^24 and a binade ends
// at most once per restart.
//
// The scan can stop at the first prefix that satisfies `acc >= bound`
// (Top-P cut) or `bound < acc` (inverse-CDF draw).
#pragma once

#include "moe_common.cuh"

namespace moe {

enum SeqStop : int
{
    kSeqSumOnly = 0,     // run to the end
    kSeqReachBound = 1,  // stop at the first i with acc >= bound
    kSeqExceedBound = 2  // stop at the first i with bound < acc
};

struct SeqResult
{
    float acc;          // accumulator after the last element taken
    uint32_t taken;     // elements added (stop element included)
    bool stopped;       // the stop condition fired
};

constexpr int kSeqHead = 256; // addends at the head of a sequence that one warp adds one by one

template<int kThreads>
struct SeqShared
{
    uint32_t warp_pair[kThreads / 32][2];
    float head[kSeqHead];   // the first addends of the sequence
    uint32_t first_event;   // smallest element offset in the chunk with a stop or a carry
    float acc;
    uint32_t stopped;
};

constexpr uint32_t kSeqSaturate = 1u << 25; // any step sum >= 2^24 means "left the binade"

__device__ __forceinline__ uint32_t seq_clamp(uint32_t v)
{
    return v < kSeqSaturate ? v : kSeqSaturate;
}

// (a then b): step sums for start parity 0 and 1
__device__ __forceinline__ void seq_compose(uint32_t a0, uint32_t a1, uint32_t b0, uint32_t b1, uint32_t& r0, uint32_t& r1)
{
    r0 = seq_clamp(a0 + ((a0 & 1u) ? b1 : b0));
    r1 = seq_clamp(a1 + (((1u + a1) & 1u) ? b1 : b0));
}

// Integer step of one non-negative addend x <= acc against the unit u of the
// accumulator, given 1/u (a power of two, so x / u is exact):
// d0 / d1 = step when the accumulator's integer is even / odd.
__device__ __forceinline__ void seq_element(float x, float inverse_unit, uint32_t& d0, uint32_t& d1)
{
    const float scaled = __fmul_rn(x, inverse_unit);          // exact; below 2^24 because x <= acc
    const uint32_t q = min(__float2uint_rz(scaled), kSeqSaturate);
    const float fraction = __fsub_rn(scaled, __uint2float_rn(q)); // exact (q < 2^24 on every path that uses it)
    const uint32_t up = fraction > 0.5f ? 1u : 0u;
    const uint32_t tie = fraction == 0.5f ? 1u : 0u;
    d0 = q + up + (tie & q);        // tie: round to the even integer
    d1 = q + up + (tie & (q + 1u));
}

// All threads of the block call this with the same arguments; x[0..n) is
// readable by every thread (global or shared).  Ends with a barrier.
// kSorted = false lifts the requirement that x does not increase (addends are
// still non-negative): an addend larger than the accumulator saturates its step
// and is handled like a binade carry, with a real add; only the early exit on
// an absorbed tail is lost.
template<int kThreads, int kItems, bool kSorted = true>
__device__ __noinline__ SeqResult block_sequential_sum(const float* x, uint32_t n, SeqStop stop, float bound, SeqShared<kThreads>& sh)
{
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u;
    const uint32_t warp = tid >> 5;
    SeqResult result{0.0f, 0u, false};
    if (n == 0)
        return result;
    // 0 + x[0] is exact
    float acc = x[0];
    uint32_t position = 1;
    if ((stop == kSeqReachBound && acc >= bound) || (stop == kSeqExceedBound && bound < acc))
    {
        result = SeqResult{acc, 1u, true};
        return result;
    }
    // The head of the sequence, literally: the first addends carry the accumulator through several
    // binades with a handful of addends each, and a round of the block (below) spends a whole chunk
    // on each of them.  One warp adds them in order, eight per trip and one test (the accumulator
    // does not decrease: a bound met by any of the eight is met by the last).
    {
        const uint32_t head = min(static_cast<uint32_t>(kSeqHead), n);
        if (tid < head)
            sh.head[tid] = x[tid];
        __syncthreads();
        if (warp == 0)
        {
            float a = acc;
            uint32_t taken = 1;
            bool stopped = false;
            while (taken < head)
            {
                const uint32_t group = min(8u, head - taken);
                float value[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    value[j] = static_cast<uint32_t>(j) < group ? sh.head[taken + j] : 0.0f; // adding +0 changes nothing
                float partial[8];
                float t = a;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    t = __fadd_rn(t, value[j]);
                    partial[j] = t;
                }
                if ((stop == kSeqReachBound && t >= bound) || (stop == kSeqExceedBound && bound < t))
                {
                    int first = 7;
#pragma unroll
                    for (int j = 6; j >= 0; --j)
                        if ((stop == kSeqReachBound && partial[j] >= bound) || (stop == kSeqExceedBound && bound < partial[j]))
                            first = j;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (j == first)
                            a = partial[j];
                    taken += static_cast<uint32_t>(first) + 1u;
                    stopped = true;
                    break;
                }
                a = t;
                taken += group;
            }
            if (lane == 0)
            {
                sh.acc = a;
                sh.first_event = taken;
                sh.stopped = stopped ? 1u : 0u;
            }
        }
        __syncthreads();
        acc = sh.acc;
        position = sh.first_event;
        const bool stopped = sh.stopped != 0;
        __syncthreads();
        if (stopped)
        {
            result = SeqResult{acc, position, true};
            return result;
        }
    }
    while (position < n)
    {
        const uint32_t acc_bits = __float_as_uint(acc);
        const int acc_biased = static_cast<int>((acc_bits >> 23) & 0xFFu);
        const uint32_t chunk = min(static_cast<uint32_t>(kThreads * kItems), n - position);
        if (acc_biased <= 23 || acc_biased == 0xFF)
        {
            // accumulator too small for a normal unit, or inf / NaN: plain adds
            // (never on the sampler's sums, whose first addend is at least 1/vocab; kept for safety)
            if (tid == 0)
            {
                float a = acc;
                uint32_t taken = position;
                uint32_t stopped = 0;
                for (uint32_t i = position; i < position + chunk; ++i)
                {
                    a = __fadd_rn(a, x[i]);
                    taken = i + 1;
                    if ((stop == kSeqReachBound && a >= bound) || (stop == kSeqExceedBound && bound < a))
                    {
                        stopped = 1;
                        break;
                    }
                }
                sh.acc = a;
                sh.first_event = taken;
                sh.stopped = stopped;
            }
            __syncthreads();
            acc = sh.acc;
            position = sh.first_event;
            const bool stopped = sh.stopped != 0;
            __syncthreads();
            if (stopped)
            {
                result = SeqResult{acc, position, true};
                return result;
            }
            continue;
        }
        const uint32_t start_integer = (acc_bits & 0x7FFFFFu) | 0x800000u;
        const float unit = __uint_as_float(static_cast<uint32_t>(acc_biased - 23) << 23); // 2^(b-23), normal because acc_biased > 23
        const float inverse_unit = __uint_as_float(static_cast<uint32_t>(277 - acc_biased) << 23); // 2^(23-b), normal for the same reason
        // The sequence does not increase and the accumulator does not decrease:
        // once the next addend is below half a unit, no later add changes the
        // accumulator (and no stop condition can fire any more).
        if (kSorted && x[position] < 0.5f * unit)
            break;

        // my kItems consecutive elements
        float mine[kItems];
        uint32_t t0 = 0, t1 = 0; // composed over my elements
        const uint32_t first = tid * kItems;
#pragma unroll
        for (int j = 0; j < kItems; ++j)
        {
            const uint32_t offset = first + j;
            mine[j] = (offset < chunk) ? x[position + offset] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < kItems; ++j)
        {
            uint32_t e0, e1;
            seq_element(mine[j], inverse_unit, e0, e1);
            if (j == 0)
            {
                t0 = e0;
                t1 = e1;
            }
            else
            {
                seq_compose(t0, t1, e0, e1, t0, t1);
            }
        }
        // inclusive scan of the thread aggregates across the warp
        uint32_t s0 = t0, s1 = t1;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1)
        {
            const uint32_t p0 = __shfl_up_sync(kFullMask, s0, offset);
            const uint32_t p1 = __shfl_up_sync(kFullMask, s1, offset);
            if (lane >= static_cast<uint32_t>(offset))
                seq_compose(p0, p1, s0, s1, s0, s1);
        }
        if (lane == 31)
        {
            sh.warp_pair[warp][0] = s0;
            sh.warp_pair[warp][1] = s1;
        }
        if (tid == 0)
        {
            sh.first_event = 0xFFFFFFFFu;
            sh.stopped = 0;
        }
        __syncthreads();
        // step sum of everything before my warp, for the actual start parity:
        // every warp scans the warps' pairs with shuffles (lane w holds warp w)
        const uint32_t start_parity = start_integer & 1u;
        uint32_t before = 0; // integer steps taken before my first element
        {
            constexpr uint32_t kWarps = kThreads / 32;
            uint32_t w0 = lane < kWarps ? sh.warp_pair[lane][0] : 0u;
            uint32_t w1 = lane < kWarps ? sh.warp_pair[lane][1] : 0u;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1)
            {
                const uint32_t p0 = __shfl_up_sync(kFullMask, w0, offset);
                const uint32_t p1 = __shfl_up_sync(kFullMask, w1, offset);
                if (lane >= static_cast<uint32_t>(offset))
                    seq_compose(p0, p1, w0, w1, w0, w1);
            }
            // inclusive pair of the warps up to warp - 1
            const uint32_t prior0 = __shfl_sync(kFullMask, w0, warp == 0 ? 0 : warp - 1);
            const uint32_t prior1 = __shfl_sync(kFullMask, w1, warp == 0 ? 0 : warp - 1);
            uint32_t parity = start_parity;
            if (warp > 0)
            {
                before = start_parity ? prior1 : prior0;
                parity = (start_parity + before) & 1u;
            }
            // lanes before me inside the warp
            const uint32_t x0 = __shfl_up_sync(kFullMask, s0, 1);
            const uint32_t x1 = __shfl_up_sync(kFullMask, s1, 1);
            if (lane > 0)
                before = seq_clamp(before + (parity ? x1 : x0));
        }
        // walk my elements with the true running integer
        uint32_t running = seq_clamp(start_integer + before);
        uint32_t event = 0xFFFFFFFFu; // first offset of mine that stops or leaves the binade
#pragma unroll
        for (int j = 0; j < kItems; ++j)
        {
            const uint32_t offset = first + j;
            if (offset < chunk && event == 0xFFFFFFFFu)
            {
                uint32_t e0, e1; // recomputed rather than kept: registers are the scarce resource here
                seq_element(mine[j], inverse_unit, e0, e1);
                const uint32_t next = seq_clamp(running + ((running & 1u) ? e1 : e0));
                if (running >= (1u << 24) || next >= (1u << 24))
                {
                    event = offset; // carry out of the binade at this element (or already before it)
                }
                else
                {
                    const float value = __uint2float_rn(next) * unit; // exact: next < 2^24, unit a power of two
                    if ((stop == kSeqReachBound && value >= bound) || (stop == kSeqExceedBound && bound < value))
                        event = offset; // `running` stays the integer before this element: its owner adds it below
                    else
                        running = next;
                }
            }
        }
        if (event != 0xFFFFFFFFu)
            atomicMin(&sh.first_event, event);
        __syncthreads();
        const uint32_t first_event = sh.first_event;
        if (first_event == 0xFFFFFFFFu)
        {
            // whole chunk inside the binade, no stop: the last thread with an element holds the final integer
            const uint32_t last_offset = chunk - 1;
            if (last_offset / kItems == tid)
                sh.acc = __uint2float_rn(running) * unit;
            __syncthreads();
            acc = sh.acc;
            position += chunk;
            __syncthreads();
            continue;
        }
        // The owner of the event element finishes it: its `running` is the exact
        // integer before that element.  Either the element stops the scan inside
        // the binade, or it is added with a real fp32 add (binade carry) and then
        // tested.
        if (first_event / kItems == tid)
        {
            const int j = static_cast<int>(first_event - first);
            float value_before = __uint2float_rn(running) * unit;
            // `running` was advanced only up to the event element because the walk stops there
            float addend = 0.0f;
#pragma unroll
            for (int k = 0; k < kItems; ++k)
                if (k == j)
                    addend = mine[k];
            const float value = __fadd_rn(value_before, addend);
            sh.acc = value;
            sh.stopped = ((stop == kSeqReachBound && value >= bound) || (stop == kSeqExceedBound && bound < value)) ? 1u : 0u;
        }
        __syncthreads();
        acc = sh.acc;
        const bool stopped = sh.stopped != 0;
        position += first_event + 1;
        __syncthreads();
        if (stopped)
        {
            result = SeqResult{acc, position, true};
            return result;
        }
    }
    result = SeqResult{acc, n, false};
    return result;
}

} // namespace moe
