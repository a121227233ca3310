// The arithmetic tail of the sampler, executed by ONE warp over candidates that
// are already in the reference rank order (logit descending, token id
// ascending).  It reproduces src/engine/session.cpp:89-136 and :429-442 step by
// step: every sum is a left-to-right fp32 accumulation in rank order, because
// the reference's results (the Top-P cut in particular) depend on that order.
// The expensive per-candidate work (exp, divisions) is done one candidate per
// lane into a scratch array; the running sums are then replayed in order by the
// whole warp (addends broadcast by shuffle, so that only the dependent adds are
// on the critical path), every lane holding the same accumulator, and the
// places where a sum crosses a bound are found with a vote.
#pragma once

#include "moe_common.cuh"

namespace moe {

struct RowOutcome
{
    int32_t status;
    int32_t token;
    float probability;
    uint32_t flags;
    // The draw ran past every candidate this warp was given although further
    // (numerically dead) candidates exist in the row: the exact path must
    // finish the row.
    bool defer;
};

// Where one row's kept candidates go (all null / 0 when the caller did not ask).
struct KeptList
{
    int32_t* token;
    float* probability;
    uint32_t* count;
    uint32_t stride;
};

__device__ __forceinline__ KeptList kept_list_of_row(int32_t* token, float* probability, uint32_t* count, uint32_t stride, uint32_t row)
{
    KeptList list{nullptr, nullptr, nullptr, 0u};
    if (count != nullptr)
    {
        list.token = token != nullptr ? token + static_cast<size_t>(row) * stride : nullptr;
        list.probability = probability != nullptr ? probability + static_cast<size_t>(row) * stride : nullptr;
        list.count = count + row;
        list.stride = stride;
    }
    return list;
}

// Left-to-right fp32 accumulation of x[0..n) (shared memory) from zero by one warp, 32
// addends per round: every lane fetches one addend, the dependent adds walk
// the lanes in order (the shuffles do not depend on the accumulator, so only
// the adds are on the critical path) and each lane keeps the accumulator as it
// stood right after its own addend.  All lanes hold the same accumulator.
enum SeqStopKind : int
{
    kSeqWarpAll = 0,    // add everything
    kSeqWarpReach = 1,  // stop behind the first addend after which acc >= bound
    kSeqWarpExceed = 2  // stop behind the first addend after which bound < acc
};

struct SeqWarpResult
{
    float acc;      // accumulator after the stopping addend, or after all n
    uint32_t index; // position of the stopping addend, n when none stopped
};

template<int kKind>
__device__ __forceinline__ SeqWarpResult warp_sequential_sum(const float* x, uint32_t n, float bound)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t addends = shared_address(x);
    float acc = 0.0f;
    for (uint32_t base = 0; base < n; base += 32)
    {
        const uint32_t i = base + lane;
        const float mine = (i < n) ? load_shared_f32(addends + 4u * i) : 0.0f;
        float after = 0.0f; // accumulator right after this lane's addend
        if (n - base >= 32u)
        {
#pragma unroll
            for (uint32_t j = 0; j < 32; ++j)
            {
                acc = __fadd_rn(acc, __shfl_sync(kFullMask, mine, j));
                after = (lane == j) ? acc : after;
            }
        }
        else
        {
            const uint32_t steps = n - base;
            for (uint32_t j = 0; j < steps; ++j)
            {
                acc = __fadd_rn(acc, __shfl_sync(kFullMask, mine, j));
                after = (lane == j) ? acc : after;
            }
        }
        if (kKind != kSeqWarpAll)
        {
            const bool stop = (i < n) && (kKind == kSeqWarpReach ? (after >= bound) : (bound < after));
            const unsigned stoppers = __ballot_sync(kFullMask, stop);
            if (stoppers != 0u)
            {
                const int first = __ffs(stoppers) - 1;
                return SeqWarpResult{__shfl_sync(kFullMask, after, first), base + static_cast<uint32_t>(first)};
            }
        }
    }
    return SeqWarpResult{acc, n};
}

// records[0..count): sorted descending.  work[0..count): scratch floats.
// tail_may_exist: the list is only the numerically live prefix of the row's
// candidates (every omitted candidate has exp(x - peak) < 2^-26, so it cannot
// change any of the four running sums, but it could still be the fall-back
// "last candidate" of session.cpp:441-442).
// numerators_ready: work[i] already holds exp(logit_i / T - peak) for every
// finite candidate the Top-K truncation leaves (computed by the whole block).
__device__ __forceinline__ RowOutcome finish_row_warp(const uint64_t* records, uint32_t count, float* work, bool numerators_ready, float temperature,
                                                       uint32_t top_k, float top_p, float min_p, float uniform, bool tail_may_exist,
                                                       const KeptList& kept_list)
{
    const int lane = threadIdx.x & 31;
    // records and work are shared memory: read through their window addresses
    const uint32_t record_base = shared_address(records);
    const uint32_t work_base = shared_address(work);
    const auto record_at = [&](uint32_t i) -> uint64_t { return load_shared_64(record_base + 8u * i); };
    const auto work_at = [&](uint32_t i) -> float { return load_shared_f32(work_base + 4u * i); };
    const auto set_work = [&](uint32_t i, float value) { store_shared_32(work_base + 4u * i, __float_as_uint(value)); };
    RowOutcome out{MOE_ROW_OK, -1, 0.0f, 0u, false};
    if (kept_list.count != nullptr && lane == 0)
        *kept_list.count = 0; // stays 0 on every error return
    if (count == 0)
    {
        out.status = MOE_ROW_NO_FINITE_LOGIT;
        return out;
    }
    const uint32_t head_key = record_key(record_at(0));
    if (head_key >= kKeyPosInf || head_key <= kKeyNegInf)
    {
        out.status = MOE_ROW_NO_FINITE_LOGIT; // session.cpp:84-85
        return out;
    }
    uint32_t considered = count;
    bool list_is_complete = !tail_may_exist;
    if (top_k > 0 && top_k <= count)
    {
        considered = top_k; // session.cpp:86-87
        list_is_complete = true;
    }
    // -inf logits sort last and are skipped (session.cpp:96-97)
    uint32_t finite = 0;
    for (uint32_t base = 0; base < considered; base += 32)
    {
        const uint32_t i = base + lane;
        const bool is_finite = (i < considered) && (record_key(record_at(i)) > kKeyNegInf);
        finite += __popc(__ballot_sync(kFullMask, is_finite));
    }

    // softmax numerators and their sequential sum (session.cpp:89-101)
    if (!numerators_ready)
    {
        const float peak = __fdiv_rn(key_to_float(head_key), temperature);
        for (uint32_t i = lane; i < finite; i += 32)
            set_work(i, exact_expf(scaled_offset(key_to_float(record_key(record_at(i))), temperature, peak)));
    }
    __syncwarp();
    const float total = warp_sequential_sum<kSeqWarpAll>(work, finite, 0.0f).acc;
    if (finite == 0 || !(total - total == 0.0f) || total <= 0.0f)
    {
        out.status = MOE_ROW_INVALID_DISTRIBUTION; // session.cpp:102-103
        return out;
    }

    // probabilities, Min-P floor, Top-P prefix (session.cpp:104-128).  The
    // reference walks the candidates once, leaving at the first one below the
    // Min-P floor or right behind the one whose running sum reaches top_p.
    // Probabilities do not increase along the list, so the candidates that pass
    // the floor are a prefix: find its length with votes, then run the
    // sequential sum over that prefix only.
    __syncwarp();
    for (uint32_t i = lane; i < finite; i += 32)
        set_work(i, __fdiv_rn(work_at(i), total));
    __syncwarp();
    uint32_t allowed = finite;
    if (min_p > 0.0f)
    {
        const float floor_probability = __fmul_rn(work_at(0), min_p);
        for (uint32_t base = 0; base < finite; base += 32)
        {
            const uint32_t i = base + lane;
            const bool below = (i < finite) && !(work_at(i) >= floor_probability);
            const unsigned voters = __ballot_sync(kFullMask, below);
            if (voters != 0u)
            {
                allowed = base + static_cast<uint32_t>(__ffs(voters) - 1);
                break;
            }
        }
    }
    const SeqWarpResult nucleus = warp_sequential_sum<kSeqWarpReach>(work, allowed, top_p);
    const uint32_t kept = nucleus.index < allowed ? nucleus.index + 1u : allowed;
    // Min-P or Top-P closed the list: no omitted candidate can follow it
    const bool cut = nucleus.index < allowed || allowed < finite;

    // renormaliser (session.cpp:130-134): the same adds over the same prefix from the same zero as the loop above
    const float kept_total = nucleus.acc;

    if (kept_list.count != nullptr && !list_is_complete && !cut)
    {
        out.defer = true; // the kept list runs on into the omitted candidates: the exact path lists them
        return out;
    }
    if (kept == 1)
    {
        out.token = static_cast<int32_t>(record_index(record_at(0))); // session.cpp:429-430: no uniform drawn
        out.probability = 1.0f;
        if (kept_list.count != nullptr && lane == 0)
        {
            *kept_list.count = 1;
            if (kept_list.stride > 0)
            {
                if (kept_list.token != nullptr)
                    kept_list.token[0] = out.token;
                if (kept_list.probability != nullptr)
                    kept_list.probability[0] = 1.0f; // x / x
            }
        }
        return out;
    }
    out.flags |= MOE_ROW_FLAG_USED_UNIFORM;

    // inverse CDF (session.cpp:432-442)
    __syncwarp();
    for (uint32_t i = lane; i < kept; i += 32)
        set_work(i, __fdiv_rn(work_at(i), kept_total));
    __syncwarp();
    if (kept_list.count != nullptr)
    {
        if (lane == 0)
            *kept_list.count = kept;
        for (uint32_t i = lane; i < min(kept, kept_list.stride); i += 32)
        {
            if (kept_list.token != nullptr)
                kept_list.token[i] = static_cast<int32_t>(record_index(record_at(i)));
            if (kept_list.probability != nullptr)
                kept_list.probability[i] = work_at(i);
        }
    }
    const SeqWarpResult draw = warp_sequential_sum<kSeqWarpExceed>(work, kept, uniform);
    if (draw.index < kept)
    {
        out.token = static_cast<int32_t>(record_index(record_at(draw.index)));
        out.probability = work_at(draw.index);
        return out;
    }
    if (!list_is_complete && !cut)
    {
        out.defer = true;
        return out;
    }
    out.token = static_cast<int32_t>(record_index(record_at(kept - 1)));
    out.probability = work_at(kept - 1);
    return out;
}

// Linear search of the row's stop list (src/engine/session.cpp:60-63).
__device__ __forceinline__ bool is_stop_token(const int32_t* stop_offsets, const int32_t* stop_tokens, uint32_t row, int32_t token)
{
    if (stop_offsets == nullptr || stop_tokens == nullptr)
        return false;
    for (int32_t i = stop_offsets[row]; i < stop_offsets[row + 1]; ++i)
        if (stop_tokens[i] == token)
            return true;
    return false;
}

} // namespace moe
