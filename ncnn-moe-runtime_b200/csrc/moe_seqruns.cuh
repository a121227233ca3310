// Block-parallel, bit-exact replay of a left-to-right fp32 accumulation over a
// sequence given as RUNS of equal addends:
//     acc = 0; for every run r in order: repeat count[r] times: acc = acc + x[r]
// with x non-increasing and non-negative — the sums of the reference sampler
// (src/engine/session.cpp:92-101,119-134,434-440) over a row of bf16 logits,
// where equal logits are equal addends and a row holds a few thousand distinct
// values instead of a hundred thousand candidates.
//
// Same arithmetic as moe_seqscan.cuh: inside one binade of the accumulator an
// addend is an integer step that depends at most on the accumulator's parity
// (exact ties of the rounding), a step is a pair (even start, odd start) and
// pairs compose associatively.  A run of c equal addends is again such a pair,
// in closed form: after a tie step the accumulator's integer is even and the
// tie step from an even integer is even, so every copy after the first takes
// the even-start step d0:
//     steps(c, parity) = (parity ? d1 : d0) + (c - 1) * d0
// (for an addend that is no tie d0 = d1 and this is c * d0).  The place inside a
// run where the accumulator leaves its binade or meets the stop condition is
// found by bisection on the copy count, because the accumulator only grows.
#pragma once

#include "moe_seqscan.cuh"


namespace moe {

struct SeqRunsResult
{
    float acc;       // accumulator after the last addend taken
    uint32_t taken;  // addends (copies, not runs) taken, the stopping one included
    bool stopped;    // the stop condition fired
    bool unsupported; // the accumulator left the range this replay handles: the caller must use another path
};

constexpr int kSeqRunsHead = 192; // addends at the head of a sequence that are added literally

template<int kThreads>
struct SeqRunsShared
{
    uint32_t warp_pair[kThreads / 32][2];
    float head_addend[kSeqRunsHead];   // the first addends of the sequence, one by one
    uint32_t head_run[kSeqRunsHead];   // ... and the run each belongs to
    uint32_t first_event; // smallest run offset in the chunk with a stop or a carry
    uint32_t event_copies; // copies of that run consumed, the event's copy included
    float acc;
    uint32_t stopped;
};

// integer steps of `copies` equal addends (pair d0 / d1) from an accumulator integer of the given parity
__device__ __forceinline__ unsigned long long seq_run_steps(uint32_t d0, uint32_t d1, uint32_t copies, uint32_t parity)
{
    if (copies == 0)
        return 0ull;
    return static_cast<unsigned long long>(parity ? d1 : d0) + static_cast<unsigned long long>(copies - 1u) * d0;
}

__device__ __forceinline__ uint32_t seq_clamp64(unsigned long long v)
{
    return v < kSeqSaturate ? static_cast<uint32_t>(v) : kSeqSaturate;
}

// Approximate inclusive prefix sums of count[r] * x[r] over the runs, by the whole block
// (plain parallel fp32 sums: a guide for the replay below, never a result).
// warp_scratch: kThreads / 32 floats of shared memory.  Ends with a barrier.
template<int kThreads, int kItems>
__device__ void block_runs_prefix_guide(const float* x, const uint32_t* count, uint32_t runs, float* prefix, float* warp_scratch)
{
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u;
    const uint32_t warp = tid >> 5;
    const uint32_t first = tid * kItems;
    float local[kItems];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < kItems; ++j)
    {
        const uint32_t r = first + j;
        if (r < runs)
            sum += static_cast<float>(count[r]) * x[r];
        local[j] = sum;
    }
    float scan = sum;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1)
    {
        const float other = __shfl_up_sync(kFullMask, scan, offset);
        if (lane >= static_cast<uint32_t>(offset))
            scan += other;
    }
    if (lane == 31)
        warp_scratch[warp] = scan;
    __syncthreads();
    float before = scan - sum;
    for (uint32_t w = 0; w < warp; ++w)
        before += warp_scratch[w];
#pragma unroll
    for (int j = 0; j < kItems; ++j)
    {
        const uint32_t r = first + j;
        if (r < runs)
            prefix[r] = before + local[j];
    }
    __syncthreads();
}

// x[r], count[r], cum[r] (= addends before run r) for r < runs, readable by every
// thread.  Only the first `limit` addends of the sequence take part.  All
// threads of the block call this with the same arguments; ends with a barrier.
//
// `guide` (optional): guide[r] * guide_scale ~ the sum of count * x over the runs 0..r
// (block_runs_prefix_guide of the same runs, possibly in other units).  A round of the
// replay covers one binade of the accumulator; with the guide it only looks at the runs
// expected to fall into that binade (plus a margin) instead of all that remain.  A guide
// that is off costs an extra round, never a different result.
template<int kThreads, int kItems>
__device__ __noinline__ SeqRunsResult block_sequential_sum_runs(const float* x, const uint32_t* count, const uint32_t* cum, uint32_t runs, uint32_t limit,
                                                                SeqStop stop, float bound, SeqRunsShared<kThreads>& sh,
                                                                const float* guide = nullptr, float guide_scale = 1.0f)
{
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u;
    const uint32_t warp = tid >> 5;
    SeqRunsResult result{0.0f, 0u, false, false};
    if (runs == 0 || limit == 0)
        return result;
    // copies of run r that take part
    const auto copies_of = [&](uint32_t r) -> uint32_t {
        const uint32_t before = cum[r];
        if (before >= limit)
            return 0u;
        return min(count[r], limit - before);
    };
    // 0 + x[0] is exact
    float acc = x[0];
    uint32_t run = 0;     // current run
    uint32_t done = 1;    // copies of it already added
    if ((stop == kSeqReachBound && acc >= bound) || (stop == kSeqExceedBound && bound < acc))
        return SeqRunsResult{acc, 1u, true, false};
    // The head of the sequence, literally: the first addends carry the accumulator through several
    // binades with a handful of addends each, where a round of the block (below) costs far more
    // than the adds themselves.  The threads lay the first addends out one by one, then one warp
    // adds them in order while the others wait.
    {
        const uint32_t total_addends = min(limit, cum[runs - 1u] + count[runs - 1u]);
        const uint32_t head = min(static_cast<uint32_t>(kSeqRunsHead), total_addends);
        if (tid < head)
        {
            // the run of addend number tid: the last run that starts at or before it (runs are not empty, so it is <= tid)
            uint32_t lo = 0, hi = min(runs - 1u, tid);
            while (lo < hi)
            {
                const uint32_t mid = lo + (hi - lo + 1u) / 2u;
                if (cum[mid] <= tid)
                    lo = mid;
                else
                    hi = mid - 1u;
            }
            sh.head_addend[tid] = x[lo];
            sh.head_run[tid] = lo;
        }
        __syncthreads();
        if (warp == 0)
        {
            float a = acc;
            uint32_t taken = 1;
            bool stopped = false;
            // eight adds per trip, then one test: the accumulator does not decrease, so a bound met by
            // any of the eight is met by the last (adding the +0 padding changes nothing)
            while (taken < head)
            {
                const uint32_t group = min(8u, head - taken);
                float value[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    value[j] = static_cast<uint32_t>(j) < group ? sh.head_addend[taken + j] : 0.0f;
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
                const uint32_t last_run = sh.head_run[taken - 1u];
                sh.acc = a;
                sh.first_event = last_run;
                sh.event_copies = taken - cum[last_run];
                sh.stopped = stopped ? 1u : 0u;
            }
        }
        __syncthreads();
        acc = sh.acc;
        run = sh.first_event;
        done = sh.event_copies;
        const bool stopped = sh.stopped != 0;
        __syncthreads();
        if (stopped)
            return SeqRunsResult{acc, cum[run] + done, true, false};
    }
    for (;;)
    {
        while (run < runs && cum[run] < limit && done >= copies_of(run))
        {
            ++run;
            done = 0;
        }
        if (run >= runs || cum[run] >= limit)
            break;
        const uint32_t acc_bits = __float_as_uint(acc);
        const int acc_biased = static_cast<int>((acc_bits >> 23) & 0xFFu);
        if (acc_biased <= 23 || acc_biased == 0xFF)
        {
            result.unsupported = true; // never on the sampler's sums (first addend >= 1 / vocab)
            return result;
        }
        const uint32_t start_integer = (acc_bits & 0x7FFFFFu) | 0x800000u;
        const float unit = __uint_as_float(static_cast<uint32_t>(acc_biased - 23) << 23);
        const float inverse_unit = __uint_as_float(static_cast<uint32_t>(277 - acc_biased) << 23);
        // the sequence does not increase and the accumulator does not decrease: once the next
        // addend is below half a unit nothing changes any more and no stop can fire
        if (x[run] < 0.5f * unit)
            break;
        uint32_t chunk = min(static_cast<uint32_t>(kThreads * kItems), runs - run);
        if (guide != nullptr)
        {
            // first run whose guide value reaches the top of this binade: every warp searches alike,
            // its lanes probing 32 places of the remaining range at a time
            const float top = 2.0f * __uint_as_float(static_cast<uint32_t>(acc_biased) << 23);
            uint32_t lo = run, hi = run + chunk; // the answer lies in [lo, hi]; guide[hi] counts as reaching
            while (lo < hi)
            {
                const uint32_t span = hi - lo;
                const uint32_t stride = (span + 31u) / 32u;
                const uint32_t probe = lo + lane * stride; // ascending over the lanes
                const bool reaches = probe >= hi || guide[probe] * guide_scale >= top;
                const unsigned votes = __ballot_sync(kFullMask, reaches);
                const uint32_t first_lane = votes != 0u ? static_cast<uint32_t>(__ffs(votes)) - 1u : 32u; // 32: beyond every probe
                hi = min(hi, lo + first_lane * stride);
                lo = first_lane == 0u ? hi : lo + (first_lane - 1u) * stride + 1u;
            }
            const uint32_t expected = lo - run + 1u;
            chunk = min(chunk, max(expected + (expected >> 5) + 8u, 64u));
        }

        // my consecutive runs of the chunk: as few per thread as the chunk allows (the round is
        // as long as one thread's work)
        const uint32_t per_thread = (chunk + kThreads - 1u) / kThreads;
        float mine[kItems];
        uint32_t copies[kItems];
        uint32_t t0 = 0, t1 = 0;
        const uint32_t first = tid * per_thread;
#pragma unroll
        for (int j = 0; j < kItems; ++j)
        {
            const uint32_t offset = first + j;
            mine[j] = 0.0f;
            copies[j] = 0;
            if (j < per_thread && offset < chunk)
            {
                mine[j] = x[run + offset];
                copies[j] = copies_of(run + offset) - (offset == 0 ? done : 0u);
            }
        }
        // threads beyond the chunk keep the identity pair (0, 0): a row has a few thousand runs at most
        if (first < chunk)
        {
#pragma unroll
            for (int j = 0; j < kItems; ++j)
            {
                if (j >= per_thread)
                    break;
                uint32_t d0, d1;
                seq_element(mine[j], inverse_unit, d0, d1);
                const uint32_t e0 = seq_clamp64(seq_run_steps(d0, d1, copies[j], 0u));
                const uint32_t e1 = seq_clamp64(seq_run_steps(d0, d1, copies[j], 1u));
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
        }
        // warps whose runs all lie beyond the chunk only keep the barriers company
        const bool warp_active = warp * 32u * per_thread < chunk;
        uint32_t s0 = t0, s1 = t1;
        if (warp_active)
        {
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1)
            {
                const uint32_t p0 = __shfl_up_sync(kFullMask, s0, offset);
                const uint32_t p1 = __shfl_up_sync(kFullMask, s1, offset);
                if (lane >= static_cast<uint32_t>(offset))
                    seq_compose(p0, p1, s0, s1, s0, s1);
            }
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
        const uint32_t start_parity = start_integer & 1u;
        uint32_t before = 0; // integer steps taken before my first run
        if (warp_active)
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
            const uint32_t prior0 = __shfl_sync(kFullMask, w0, warp == 0 ? 0 : warp - 1);
            const uint32_t prior1 = __shfl_sync(kFullMask, w1, warp == 0 ? 0 : warp - 1);
            uint32_t parity = start_parity;
            if (warp > 0)
            {
                before = start_parity ? prior1 : prior0;
                parity = (start_parity + before) & 1u;
            }
            const uint32_t x0 = __shfl_up_sync(kFullMask, s0, 1);
            const uint32_t x1 = __shfl_up_sync(kFullMask, s1, 1);
            if (lane > 0)
                before = seq_clamp(before + (parity ? x1 : x0));
        }
        // walk my runs with the true running integer
        uint32_t running = seq_clamp(start_integer + before);
        uint32_t event = 0xFFFFFFFFu; // first offset of mine inside which the scan stops or leaves the binade
#pragma unroll
        for (int j = 0; j < kItems; ++j)
        {
            const uint32_t offset = first + j;
            if (j < per_thread && offset < chunk && event == 0xFFFFFFFFu && copies[j] != 0u)
            {
                uint32_t d0, d1;
                seq_element(mine[j], inverse_unit, d0, d1);
                const uint32_t next = seq_clamp64(running + seq_run_steps(d0, d1, copies[j], running & 1u));
                if (running >= (1u << 24) || next >= (1u << 24))
                {
                    event = offset;
                }
                else
                {
                    const float value = __uint2float_rn(next) * unit; // exact
                    if ((stop == kSeqReachBound && value >= bound) || (stop == kSeqExceedBound && bound < value))
                        event = offset; // the accumulator only grows: the first copy that satisfies the bound is inside this run
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
            // the whole chunk inside the binade, no stop: the thread that owns the last run holds the final integer
            const uint32_t last_offset = chunk - 1;
            if (last_offset / per_thread == tid)
                sh.acc = __uint2float_rn(running) * unit;
            __syncthreads();
            acc = sh.acc;
            run += chunk;
            done = 0;
            __syncthreads();
            continue;
        }
        if (first_event / per_thread == tid)
        {
            // `running` is the exact integer before the event run.  Find the first copy m (1-based)
            // after which the integer has left the binade or the bound is met.
            const int j = static_cast<int>(first_event - first);
            float addend = 0.0f;
            uint32_t available = 0;
#pragma unroll
            for (int k = 0; k < kItems; ++k)
                if (k == j)
                {
                    addend = mine[k];
                    available = copies[k];
                }
            uint32_t d0, d1;
            seq_element(addend, inverse_unit, d0, d1);
            const uint32_t parity = running & 1u;
            const auto is_event = [&](uint32_t m) -> bool {
                const unsigned long long integer = running + seq_run_steps(d0, d1, m, parity);
                if (integer >= (1ull << 24))
                    return true;
                const float value = __uint2float_rn(static_cast<uint32_t>(integer)) * unit;
                return (stop == kSeqReachBound && value >= bound) || (stop == kSeqExceedBound && bound < value);
            };
            uint32_t lo = 1, hi = available; // is_event(available) holds
            while (lo < hi)
            {
                const uint32_t mid = lo + (hi - lo) / 2u;
                if (is_event(mid))
                    hi = mid;
                else
                    lo = mid + 1u;
            }
            const uint32_t m = lo;
            const unsigned long long integer_before = running + seq_run_steps(d0, d1, m - 1u, parity);
            const unsigned long long integer_after = running + seq_run_steps(d0, d1, m, parity);
            float value;
            if (integer_after >= (1ull << 24))
            {
                // the m-th copy carries out of the binade: a real fp32 add from the exact value before it
                const float value_before = __uint2float_rn(static_cast<uint32_t>(integer_before)) * unit;
                value = __fadd_rn(value_before, addend);
            }
            else
            {
                value = __uint2float_rn(static_cast<uint32_t>(integer_after)) * unit;
            }
            sh.acc = value;
            sh.event_copies = m;
            sh.stopped = ((stop == kSeqReachBound && value >= bound) || (stop == kSeqExceedBound && bound < value)) ? 1u : 0u;
        }
        __syncthreads();
        acc = sh.acc;
        const bool stopped = sh.stopped != 0;
        const uint32_t consumed = sh.event_copies;
        done = (first_event == 0 ? done : 0u) + consumed;
        run += first_event;
        __syncthreads();
        if (stopped)
            return SeqRunsResult{acc, cum[run] + done, true, false};
    }
    return SeqRunsResult{acc, limit, false, false};
}

} // namespace moe
