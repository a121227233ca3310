// Verification step of speculative decoding, one CTA per Session
// (src/engine/session.cpp:776-880): walk the proposed tokens, accept each with
// probability min(1, p_target / p_draft) (:800-835), and produce the token
// that follows the accepted prefix — a draw from the residual distribution
// max(0, target - draft) after a rejection (sample_residual_distribution,
// :150-202), else the sample of the next target row.
//
// The distributions come from the sampler kernels (kept-candidate lists, the
// vectors sampling_distribution returns); this kernel is the control flow on
// top of them.  One CTA per Session: the walk is sequential by nature (position j is only
// looked at when 0..j-1 were accepted), the look-ups and the residual are
// spread over the threads.  The residual sums run in token-id order like the
// reference's std::accumulate over its dense vector; zeros change nothing in
// an fp32 sum, so only the positive entries are added, in that order.

#include "moe_common.cuh"
#include "moe_internal.h"
#include "moe_seqscan.cuh"

namespace moe {

namespace {

constexpr int kVerifyThreads = 1024;
constexpr int kVerifyWarps = kVerifyThreads / 32;

struct VerifyShared
{
    SeqShared<kVerifyThreads> seq;
    float found[2];
    uint32_t warp_count[kVerifyWarps];
    uint32_t cursor;
    uint32_t decision; // 0 accepted, 1 rejected, 2 error
};

// candidate_probability (session.cpp:138-148): the probability listed for `token`, 0 if absent.
// Token ids are unique in a list, so at most one thread writes.
__device__ float list_probability(const int32_t* tokens, const float* probabilities, uint32_t count, int32_t token, float* slot)
{
    if (threadIdx.x == 0)
        *slot = 0.0f;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < count; i += kVerifyThreads)
        if (tokens[i] == token)
            *slot = probabilities[i];
    __syncthreads();
    return *slot;
}

} // namespace

__global__ void __launch_bounds__(kVerifyThreads, 1) speculative_verify_kernel(const SpeculativeArgs s)
{
    __shared__ VerifyShared sh;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t n = s.draft_count;
    const uint32_t session = blockIdx.x;
    // rows of the sampler outputs: every Session's draft_count + 1 target positions first, then every Session's draft positions
    const uint32_t target_first = session * (n + 1u);
    const uint32_t draft_first = s.sessions * (n + 1u) + session * n;
    const moe_row_params p = s.params[target_first];
    const int32_t* const proposed_tokens = s.proposed + static_cast<size_t>(session) * n;
    float* const accepted_probability = s.accepted_probability + static_cast<size_t>(session) * n;
    float* const dense = s.dense + static_cast<size_t>(session) * s.vocab;
    int32_t* const residual_token = s.residual_token + static_cast<size_t>(session) * s.vocab;
    float* const residual_value = s.residual_value + static_cast<size_t>(session) * s.vocab;
    const bool greedy = p.temperature == 0.0f;

    uint32_t accepted = 0;
    uint32_t used = 0;
    int32_t status = MOE_ROW_OK;
    bool rejected = false;
    while (accepted < n)
    {
        const uint32_t target_row = target_first + accepted;
        const uint32_t draft_row = draft_first + accepted;
        const int32_t proposed = proposed_tokens[accepted];
        if (s.row_status[target_row] != MOE_ROW_OK)
        {
            status = s.row_status[target_row];
            break;
        }
        if (greedy)
        {
            if (s.token[target_row] != proposed)
                break; // session.cpp:790-794
            if (tid == 0)
                accepted_probability[accepted] = 1.0f;
        }
        else
        {
            if (s.row_status[draft_row] != MOE_ROW_OK)
            {
                status = s.row_status[draft_row];
                break;
            }
            const size_t stride = s.kept_stride;
            const float target_probability = list_probability(s.kept_token + target_row * stride, s.kept_probability + target_row * stride,
                                                              min(s.kept_count[target_row], s.kept_stride), proposed, &sh.found[0]);
            const float draft_probability = list_probability(s.kept_token + draft_row * stride, s.kept_probability + draft_row * stride,
                                                             min(s.kept_count[draft_row], s.kept_stride), proposed, &sh.found[1]);
            if (!(draft_probability > 0.0f))
            {
                status = MOE_ROW_DRAFT_ZERO_PROBABILITY; // session.cpp:813-821
                break;
            }
            const float ratio = __fdiv_rn(target_probability, draft_probability);
            const float acceptance = ratio < 1.0f ? ratio : 1.0f; // std::min(1.0f, ratio)
            const float uniform = philox_uniform(p.seed, p.row_id, p.step + used);
            ++used;
            if (uniform >= acceptance)
            {
                rejected = true; // session.cpp:827-833
                break;
            }
            if (tid == 0)
                accepted_probability[accepted] = target_probability;
        }
        ++accepted;
    }

    int32_t next_token = -1;
    float next_probability = 0.0f;
    if (status == MOE_ROW_OK && rejected)
    {
        // ---- residual distribution of the rejected position (session.cpp:150-202) ----
        const uint32_t target_row = target_first + accepted;
        const uint32_t draft_row = draft_first + accepted;
        const size_t stride = s.kept_stride;
        const int32_t* target_token = s.kept_token + target_row * stride;
        const float* target_probability = s.kept_probability + target_row * stride;
        const int32_t* draft_token = s.kept_token + draft_row * stride;
        const float* draft_probability = s.kept_probability + draft_row * stride;
        const uint32_t target_count = min(s.kept_count[target_row], s.kept_stride);
        const uint32_t draft_count = min(s.kept_count[draft_row], s.kept_stride);
        for (uint32_t i = tid; i < s.vocab; i += kVerifyThreads)
            dense[i] = 0.0f;
        __syncthreads();
        for (uint32_t i = tid; i < target_count; i += kVerifyThreads)
            dense[target_token[i]] = target_probability[i];
        __syncthreads();
        for (uint32_t i = tid; i < draft_count; i += kVerifyThreads)
        {
            const int32_t id = draft_token[i];
            const float reduced = __fsub_rn(dense[id], draft_probability[i]);
            dense[id] = reduced > 0.0f ? reduced : 0.0f; // std::max(0.0f, ...)
        }
        if (tid == 0)
            sh.cursor = 0;
        __syncthreads();
        // positive entries in token-id order
        for (uint32_t base = 0; base < s.vocab; base += kVerifyThreads)
        {
            const uint32_t id = base + tid;
            const float value = id < s.vocab ? dense[id] : 0.0f;
            const bool positive = value > 0.0f;
            const unsigned voters = __ballot_sync(kFullMask, positive);
            if (lane == 0)
                sh.warp_count[warp] = __popc(voters);
            __syncthreads();
            uint32_t before = sh.cursor;
            for (int w = 0; w < warp; ++w)
                before += sh.warp_count[w];
            if (positive)
            {
                const uint32_t slot = before + __popc(voters & ((1u << lane) - 1u));
                residual_token[slot] = static_cast<int32_t>(id);
                residual_value[slot] = value;
            }
            __syncthreads();
            if (tid == kVerifyThreads - 1)
                sh.cursor = before + __popc(voters);
            __syncthreads();
        }
        const uint32_t positives = sh.cursor;
        __syncthreads();
        // std::accumulate over the dense vector (session.cpp:171-176) = the positive entries added in token-id
        // order; replayed bit-exactly by the whole block (the entries are not sorted by value)
        const float normalizer = block_sequential_sum<kVerifyThreads, 8, false>(residual_value, positives, kSeqSumOnly, 0.0f, sh.seq).acc;
        if (positives == 0 || !(normalizer - normalizer == 0.0f) || normalizer <= 0.0f)
        {
            if (tid == 0)
            {
                sh.decision = 2;
                sh.found[0] = 0.0f;
                sh.cursor = 0;
            }
        }
        else
        {
            const float uniform = philox_uniform(p.seed, p.row_id, p.step + used);
            const float sample_value = __fmul_rn(uniform, normalizer); // uniform_real_distribution<float>(0, normalizer)
            const SeqResult draw = block_sequential_sum<kVerifyThreads, 8, false>(residual_value, positives, kSeqExceedBound, sample_value, sh.seq);
            // session.cpp:189-197: the last positive entry if the sum never passes the draw
            const uint32_t chosen = draw.stopped ? draw.taken - 1u : positives - 1u;
            if (tid == 0)
            {
                sh.decision = 0;
                sh.cursor = static_cast<uint32_t>(residual_token[chosen]);
                sh.found[0] = __fdiv_rn(residual_value[chosen], normalizer);
            }
        }
        __syncthreads();
        ++used;
        if (sh.decision == 2)
        {
            status = MOE_ROW_RESIDUAL_EMPTY;
            --used; // the reference returns before it draws
        }
        else
        {
            next_token = static_cast<int32_t>(sh.cursor);
            next_probability = sh.found[0];
        }
    }
    else if (status == MOE_ROW_OK)
    {
        // every proposal accepted, or greedy: the sample of the next target row (session.cpp:871-874);
        // its uniform is number `used` of this step, which is draft_count when all were accepted
        const uint32_t row = target_first + accepted;
        status = s.row_status[row];
        if (status == MOE_ROW_OK)
        {
            next_token = s.token[row];
            next_probability = s.probability[row];
            if (s.row_flags[row] & MOE_ROW_FLAG_USED_UNIFORM)
                ++used;
        }
    }
    if (tid == 0)
    {
        moe_speculative_result result;
        result.accepted = accepted;
        result.next_token = next_token;
        result.next_probability = next_probability;
        result.uniforms_used = used;
        result.status = status;
        result.flags = 0;
        s.result[session] = result;
    }
}

cudaError_t launch_speculative_verify(const SpeculativeArgs& args, cudaStream_t stream)
{
    speculative_verify_kernel<<<args.sessions, kVerifyThreads, 0, stream>>>(args);
    return cudaGetLastError();
}

} // namespace moe
