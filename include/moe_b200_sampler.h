/*
 * moe_b200_sampler.h — C ABI of the B200 (sm_100a) generation sampler and MoE
 * router Top-K.  Plain C, opaque handle, integer status per call and per row,
 * caller-owned buffers, no exceptions.  Every entry point below names the
 * reference interface it stands in for (paths are relative to the
 * ncnn-MoE-Runtime source tree).
 *
 * Threading: a handle serialises nothing.  Use one handle per host thread /
 * CUDA stream; calls on one handle must be issued in stream order on a single
 * stream because they share the handle's device workspace.
 *
 * There is no CPU fallback: every function that computes requires a CUDA
 * device of compute capability 10.x and fails with MOE_STATUS_CUDA_ERROR
 * otherwise.
 */
#ifndef MOE_B200_SAMPLER_H
#define MOE_B200_SAMPLER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Call status.  Values 1..5 are ErrorCode + 1 of include/ncnn/moe/result.h:12-19. */
enum moe_status
{
    MOE_STATUS_OK = 0,
    MOE_STATUS_INVALID_ARGUMENT = 1,
    MOE_STATUS_IO_ERROR = 2,
    MOE_STATUS_INVALID_MODEL = 3,
    MOE_STATUS_UNSUPPORTED_MODEL = 4,
    MOE_STATUS_INTERNAL_ERROR = 5,
    MOE_STATUS_CUDA_ERROR = 6
};

/* Per-row result code written to `row_status`.  1..6 carry the fixed messages
 * of src/engine/session.cpp:67-72,85,103,399,421; moe_row_status_message()
 * returns the text and moe_row_status_error_code() the ErrorCode + 1. */
enum moe_row_status
{
    MOE_ROW_OK = 0,
    MOE_ROW_EMPTY_LOGITS = 1,        /* "cannot sample empty logits" */
    MOE_ROW_BAD_TEMPERATURE = 2,     /* "temperature must be finite and non-negative" */
    MOE_ROW_BAD_TOP_P = 3,           /* "top_p must be in the range (0, 1]" */
    MOE_ROW_BAD_MIN_P = 4,           /* "min_p must be in the range [0, 1]" */
    MOE_ROW_NO_FINITE_LOGIT = 5,     /* "sampling requires at least one finite logit" */
    MOE_ROW_INVALID_DISTRIBUTION = 6,/* "sampling distribution is invalid" */
    MOE_ROW_WORKSPACE_EXHAUSTED = 7, /* library limit, no reference counterpart */
    /* speculative verification only (ErrorCode::InternalError in the reference) */
    MOE_ROW_DRAFT_ZERO_PROBABILITY = 8, /* "sampled draft token has zero probability", session.cpp:813-821 */
    MOE_ROW_RESIDUAL_EMPTY = 9          /* "speculative residual distribution is empty", session.cpp:169-174 */
};

enum moe_dtype
{
    MOE_DTYPE_F32 = 0,
    MOE_DTYPE_BF16 = 1 /* widened exactly (bits << 16), src/kernels/cpu_bfloat16.cpp:26-28 */
};

/* Bits of the per-row `row_flags` output. */
#define MOE_ROW_FLAG_STOP_TOKEN 1u   /* StreamToken::is_stop_token, include/ncnn/moe/session.h:63-72 */
#define MOE_ROW_FLAG_USED_UNIFORM 2u /* the reference would have advanced its RNG (session.cpp:429-433) */

/* Largest top_k served by the shared-memory radix select; larger values (and
 * top_k = 0) take the exact full-vocabulary path. */
#define MOE_SAMPLER_TOPK_FAST_MAX 1024u

/* One row = one Session's SamplingOptions (include/ncnn/moe/session.h:49-55)
 * plus the counter-based RNG coordinates that replace the Session's private
 * std::mt19937_64 (session.h:303; session.cpp:291,432-433).  The uniform of a
 * row is Philox4x32-10 with key = seed, counter = (row_id, step + step_offset):
 * u = (word0 >> 8) * 2^-24. */
typedef struct moe_row_params
{
    float temperature; /* 0 = greedy */
    uint32_t top_k;    /* 0 = off */
    float top_p;       /* (0, 1] */
    float min_p;       /* [0, 1] */
    uint64_t seed;
    uint64_t row_id;
    uint64_t step;
} moe_row_params;

typedef struct moe_sampler moe_sampler;

/* ---- lifetime ----------------------------------------------------------- */

/* Allocates the device workspace for batches of up to max_rows rows of up to
 * max_vocab logits on CUDA device `device`.  No reference counterpart (the
 * reference sampler is stateless apart from Session::random_generator_). */
int moe_sampler_create(int device, uint32_t max_rows, uint32_t max_vocab, moe_sampler** out);
void moe_sampler_destroy(moe_sampler* sampler);
/* Back-to-back sampling calls on one stream normally run one after the other.
 * With overlap enabled, moe_sample_batch launches its kernel with programmatic
 * stream serialization: its CTAs may take the SM slots the previous sampling
 * kernel of the stream leaves free and read their logits while that kernel is
 * still running, and they wait for it to complete before they write anything.
 * Results are unchanged.  Enable it only when the logits of a call do not
 * depend on the kernel launched immediately before it on the same stream
 * (independent batches, or logits produced earlier): that kernel is not waited
 * for before the logits are read.  Off by default.  No reference counterpart
 * (the reference samples on the host). */
int moe_sampler_set_overlap(moe_sampler* sampler, int enable);
/* Text of the last failing call on this handle (never NULL). */
const char* moe_sampler_last_error(const moe_sampler* sampler);

const char* moe_row_status_message(int row_status);
int moe_row_status_error_code(int row_status);

/* The uniform a row would consume, computed on the host (same Philox as the
 * kernels).  Replaces drawing from Session::random_generator_
 * (src/engine/session.cpp:432-433). */
float moe_philox_uniform(uint64_t seed, uint64_t row_id, uint64_t step);

/* Page-locked host memory for callers that stage logits themselves. */
int moe_host_alloc(size_t bytes, void** out);
void moe_host_free(void* pointer);

/* ---- batched sampling --------------------------------------------------- */

/* Replaces, for `rows` Sessions at once, the caller-side loop of
 * examples/internal/run_model.cpp:776-809: one Session::sample
 * (include/ncnn/moe/session.h:326; src/engine/session.cpp:393-443) per row
 * with that row's options, then the stop-token test of run_model.cpp:790.
 *
 * logits            device, [rows x row_stride] elements of `dtype`, vocab <= row_stride
 * params            HOST array of `rows` entries, or NULL to reuse the parameters
 *                   uploaded by the previous call on this handle (same row count)
 * step_offset       added to every row's `step` (lets resident parameters serve
 *                   consecutive decode steps)
 * stop_offsets      HOST, rows + 1 entries (CSR) or NULL; stop_tokens HOST or NULL
 *                   (GenerationOptions::stop_tokens, session.h:78); reused with params
 * token_id, probability  device, rows entries (SampledToken, session.h:57-61)
 * row_flags, row_status  device, rows entries (may be NULL)
 * topk_index        device, [rows x topk_stride] or NULL: for rows with
 *                   0 < top_k <= MOE_SAMPLER_TOPK_FAST_MAX the first min(top_k, topk_stride)
 *                   token ids of the reference rank order (session.cpp:80-87), -1 padded;
 *                   every other row (greedy, top_k = 0, top_k above the limit, rejected) is all -1
 * Asynchronous on `stream` (a cudaStream_t). */
int moe_sample_batch(moe_sampler* sampler, void* stream, const void* logits, int dtype, uint32_t rows, uint32_t vocab,
                     size_t row_stride, const moe_row_params* params, uint64_t step_offset, const int32_t* stop_offsets,
                     const int32_t* stop_tokens, int32_t* token_id, float* probability, uint32_t* row_flags,
                     int32_t* row_status, int32_t* topk_index, uint32_t topk_stride);

/* moe_sample_batch with its outputs in a struct, plus one more: every row's
 * kept candidates with their renormalised probabilities, i.e. the vector that
 * sampling_distribution returns (src/engine/session.cpp:76-136) and that the
 * speculative-decoding acceptance test reads through candidate_probability
 * (session.cpp:138-148,800-812).  All pointers are device pointers.
 * kept_count   [rows] or NULL: candidates kept after Top-K, Min-P and Top-P
 *              (0 for a rejected row; 1 for a greedy row, which lists its token
 *              with probability 1).  NULL switches the two lists off.
 * kept_token, kept_probability  [rows x kept_stride] or NULL: the first
 *              min(kept_count, kept_stride) candidates in rank order; entries
 *              past that are left untouched. */
typedef struct moe_sample_outputs
{
    int32_t* token_id;
    float* probability;
    uint32_t* row_flags;
    int32_t* row_status;
    int32_t* topk_index;
    uint32_t topk_stride;
    int32_t* kept_token;
    float* kept_probability;
    uint32_t* kept_count;
    uint32_t kept_stride;
} moe_sample_outputs;

int moe_sample_batch_ex(moe_sampler* sampler, void* stream, const void* logits, int dtype, uint32_t rows, uint32_t vocab,
                        size_t row_stride, const moe_row_params* params, uint64_t step_offset, const int32_t* stop_offsets,
                        const int32_t* stop_tokens, const moe_sample_outputs* outputs);

/* Sampling with the logits already on the device and only the sampled tokens
 * returned to the host: the LogitsOutputMode::SampledToken the reference
 * reserves but still rejects (include/ncnn/moe/types.h:304-309,
 * src/engine/runtime.cpp:579-580).  The staged [sessions x vocab] logit matrix
 * of the LM head (src/engine/cpu_executor.cpp:2978-2995) stays where it was
 * produced; what crosses to the host is one 16-byte record per row.
 *
 * Same arguments as moe_sample_batch up to stop_tokens.  `stream` is the stream
 * the logits were produced on: the kernel is ordered behind the producer there.
 * results   HOST (page-locked for speed: moe_host_alloc), rows records; valid when
 *           the call returns (it synchronises `stream`). */
typedef struct moe_sampled_row
{
    int32_t token_id;    /* SampledToken::token_id, -1 for a rejected row */
    float probability;   /* SampledToken::probability */
    uint32_t row_flags;  /* MOE_ROW_FLAG_* */
    int32_t row_status;  /* MOE_ROW_* */
} moe_sampled_row;

int moe_sample_tokens(moe_sampler* sampler, void* stream, const void* logits, int dtype, uint32_t rows, uint32_t vocab,
                      size_t row_stride, const moe_row_params* params, uint64_t step_offset, const int32_t* stop_offsets,
                      const int32_t* stop_tokens, moe_sampled_row* results);

/* The verification step of speculative decoding for one Session
 * (the loop of Session::generate, src/engine/session.cpp:776-880): the
 * `draft_count` proposed tokens are walked in order, each accepted with
 * probability min(1, p_target / p_draft) where both probabilities come from
 * sampling_distribution of that position's target and draft logits under the
 * Session's options (candidate_probability, :138-148); temperature 0 accepts
 * while the target's greedy token equals the proposal (:778-794).  The token
 * after the accepted prefix is a draw from the residual distribution
 * max(0, target - draft) of the rejected position, summed in token-id order
 * (sample_residual_distribution, :150-202), or the ordinary sample of the next
 * target row when nothing was rejected or temperature is 0 (:871-874).
 * Uniforms are Philox(seed, row_id, step), step advancing by one per consumed
 * uniform exactly as the Session's generator would advance.
 *
 * target_logits   device, [(draft_count + 1) x row_stride] of `dtype`
 * draft_logits    device, [draft_count x row_stride]
 * proposed_tokens device, draft_count token ids
 * params          HOST, ONE entry: the Session's options and its (seed, row_id, step)
 * accepted_probability  device, draft_count floats: the probability reported
 *                 for each accepted token (target probability; 1 when greedy)
 * result          device
 * draft_count <= MOE_SPECULATIVE_MAX_DRAFT and 2 * draft_count + 1 <= the
 * handle's max_rows.  The call replaces the handle's resident row parameters
 * and allocates its scratch on first use.  Asynchronous on `stream`. */
#define MOE_SPECULATIVE_MAX_DRAFT 16u
typedef struct moe_speculative_result
{
    uint32_t accepted;       /* proposed tokens accepted, 0..draft_count */
    int32_t next_token;      /* the token emitted after them, -1 on error */
    float next_probability;
    uint32_t uniforms_used;  /* add to the Session's step */
    int32_t status;          /* MOE_ROW_OK or the status of the position that failed */
    uint32_t flags;          /* reserved, 0 */
} moe_speculative_result;

int moe_speculative_verify(moe_sampler* sampler, void* stream, const void* target_logits, const void* draft_logits, int dtype,
                           uint32_t draft_count, uint32_t vocab, size_t row_stride, const int32_t* proposed_tokens,
                           const moe_row_params* params, float* accepted_probability, moe_speculative_result* result);

/* moe_speculative_verify for `sessions` Sessions in one call: the scheduler's
 * batch of Sessions that all verify `draft_count` proposals this step.  One
 * sampler launch covers every target position, one every draft position, and
 * one verification kernel walks the Sessions side by side (one CTA each); each
 * Session's outcome is what moe_speculative_verify gives for it alone.
 *
 * target_logits   device, [sessions x (draft_count + 1) x row_stride], Session-major
 * draft_logits    device, [sessions x draft_count x row_stride]
 * proposed_tokens device, [sessions x draft_count]
 * params          HOST, one entry per Session
 * accepted_probability  device, [sessions x draft_count]
 * results         device, [sessions]
 * sessions * (2 * draft_count + 1) <= the handle's max_rows. */
int moe_speculative_verify_batch(moe_sampler* sampler, void* stream, const void* target_logits, const void* draft_logits, int dtype,
                                 uint32_t sessions, uint32_t draft_count, uint32_t vocab, size_t row_stride, const int32_t* proposed_tokens,
                                 const moe_row_params* params, float* accepted_probability, moe_speculative_result* results);

/* moe_speculative_verify with every buffer in HOST memory (the reference holds
 * target and draft logits as std::vector<float>, session.cpp:760-769).  Copies
 * in, verifies, copies out and synchronises before returning. */
int moe_speculative_verify_host(moe_sampler* sampler, const void* target_logits, const void* draft_logits, int dtype, uint32_t draft_count,
                                uint32_t vocab, size_t row_stride, const int32_t* proposed_tokens, const moe_row_params* params,
                                float* accepted_probability, moe_speculative_result* result);

/* Same operation with every buffer in HOST memory (what a Session-shaped
 * caller holds: LogitsOutput::values is a std::vector<float>, session.h:30-33).
 * Copies in, samples, copies out and synchronises before returning. */
int moe_sample_batch_host(moe_sampler* sampler, const void* logits, int dtype, uint32_t rows, uint32_t vocab, size_t row_stride,
                          const moe_row_params* params, const int32_t* stop_offsets, const int32_t* stop_tokens,
                          int32_t* token_id, float* probability, uint32_t* row_flags, int32_t* row_status,
                          int32_t* topk_index, uint32_t topk_stride);

/* ---- vocabulary-sharded sampling ---------------------------------------- */

/* Step 1 on every GPU: the stable Top-K of this GPU's vocabulary slice
 * (src/engine/session.cpp:80-87 restricted to [vocab_begin, vocab_begin + vocab)).
 * candidates: device, [rows x top_k] 64-bit records, best first:
 *   (ordered_logit_bits << 32) | (0xFFFFFFFF - global_token_id); 0 = empty slot. */
int moe_sample_local_candidates(moe_sampler* sampler, void* stream, const void* logits, int dtype, uint32_t rows, uint32_t vocab,
                                size_t row_stride, uint32_t vocab_begin, uint32_t top_k, uint64_t* candidates);

/* Step 2 after the caller's all-gather: `gathered` is device,
 * [shards x rows x top_k] records; merges them to the global stable Top-K and
 * finishes session.cpp:89-136,429-442 on it.  Requires 0 < top_k <=
 * MOE_SAMPLER_TOPK_FAST_MAX for every row and temperature > 0. */
int moe_sample_merge_candidates(moe_sampler* sampler, void* stream, const uint64_t* gathered, uint32_t shards, uint32_t rows,
                                uint32_t top_k, const moe_row_params* params, uint64_t step_offset, int32_t* token_id,
                                float* probability, uint32_t* row_flags, int32_t* row_status, int32_t* topk_index,
                                uint32_t topk_stride);

/* ---- MoE router ---------------------------------------------------------- */

enum moe_router_score
{
    MOE_ROUTER_SOFTMAX = 0,
    MOE_ROUTER_SIGMOID = 1,
    MOE_ROUTER_SQRT_SOFTPLUS = 2 /* RouterScoreFunction, include/ncnn/moe/types.h:216-221 */
};

#define MOE_ROUTER_FLAG_NORMALIZE_TOPK 1u /* ExpertDispatchNormalizeTopKWeights, expert_dispatcher.h:27-32 */

/* ExpertDispatchOptions (include/ncnn/moe/expert_dispatcher.h:34-44). */
typedef struct moe_router_options
{
    uint32_t expert_count;
    uint32_t top_k;
    int32_t score_function;      /* moe_router_score */
    int32_t normalization;       /* 0 None, 1 SelectedExperts (types.h:223-227) */
    float routed_scaling_factor;
    uint32_t flags;
    const float* selection_bias;       /* device, expert_count entries, or NULL */
    const uint32_t* explicit_expert_ids; /* device, token_count * top_k entries, or NULL */
} moe_router_options;

/* Replaces ExpertDispatcher::dispatch / dispatch_into
 * (include/ncnn/moe/expert_dispatcher.h:57-60; src/graph/expert_dispatcher.cpp:79-301).
 * The ExpertDispatchPlan comes back as CSR arrays (all device):
 *   expert_offsets[expert_count + 1]  routes of expert e are [offsets[e], offsets[e+1])
 *   route_token / route_rank / route_weight [token_count * top_k]  ExpertRoute fields,
 *     experts ascending, inside an expert token ascending then rank ascending
 *   plan_status[1]  0, or a router status value (see moe_router_status_message)
 * Asynchronous on `stream`; the shape checks that need no data are done on the
 * host and returned directly. */
int moe_router_dispatch(moe_sampler* sampler, void* stream, const float* router_logits, uint32_t token_count,
                        const moe_router_options* options, uint32_t* expert_offsets, uint32_t* route_token,
                        uint32_t* route_rank, float* route_weight, int32_t* plan_status);
/* plan_status values: 0, or 101.. with the reference's fixed messages
 * (expert_dispatcher.cpp:81-101,128,136-137); moe_router_status_error_code()
 * maps them to ErrorCode + 1.  moe_router_check_options() runs the checks that
 * need no data (token count, top_k range, scaling factor) and returns such a
 * value. */
const char* moe_router_status_message(int plan_status);
int moe_router_status_error_code(int plan_status);
int moe_router_check_options(uint32_t token_count, const moe_router_options* options);

/* Host-buffer form of the same call (router logits are a host span in the
 * reference).  Synchronous. */
int moe_router_dispatch_host(moe_sampler* sampler, const float* router_logits, uint32_t token_count,
                             const moe_router_options* options_with_host_pointers, uint32_t* expert_offsets,
                             uint32_t* route_token, uint32_t* route_rank, float* route_weight, int32_t* plan_status);

/* Router dispatch for hosts that must not allocate device memory when they
 * route: engines whose planner or pool owns every byte of the GPU from start-up,
 * so that a late cudaMalloc fails or falsifies the planner's books, and decode
 * loops that cannot take the device-wide synchronisation an allocation may
 * cause.  It has no counterpart in the reference (whose dispatcher runs on the
 * host); it is moe_router_dispatch with its scratch held in a fixed array inside
 * the library's device image instead of grown on demand, so it needs no handle
 * and calls no allocator of any kind.
 *
 * Limits: token_count * top_k <= MOE_ROUTER_STATIC_MAX_ROUTES and expert_count
 * <= MOE_ROUTER_STATIC_MAX_EXPERTS; anything larger is refused with
 * MOE_STATUS_INVALID_ARGUMENT and a message in error_text.  The array costs
 * MOE_ROUTER_STATIC_SCRATCH_BYTES on every GPU that loads the library, until
 * the process ends.
 *
 * It works on the CURRENT device.  The first call on a device looks the
 * array's address up (cudaGetSymbolAddress); make that first call during
 * start-up, before any stream capture begins.  All calls share the one array:
 * each call resets the counters it needs, but two calls that overlap on the GPU
 * (different streams, or several host threads) race on it — keep them
 * stream-ordered.
 *
 * All pointers are device pointers (options->selection_bias /
 * explicit_expert_ids too); outputs are as for moe_router_dispatch.
 * error_text may be NULL. */
#define MOE_ROUTER_STATIC_MAX_ROUTES 65536u
#define MOE_ROUTER_STATIC_MAX_EXPERTS 4096u
#define MOE_ROUTER_STATIC_SCRATCH_BYTES (1568u * 1024u)
int moe_router_dispatch_static(void* stream, const float* router_logits, uint32_t token_count,
                               const moe_router_options* options, uint32_t* expert_offsets, uint32_t* route_token,
                               uint32_t* route_rank, float* route_weight, int32_t* plan_status, char* error_text,
                               size_t error_capacity);

/* Replaces gather_tokens (src/engine/cpu_executor.cpp:635-642): copies
 * hidden[route_token[i], :] to gathered[i, :] for every route.  All device.
 * A route_token entry >= token_count is never dereferenced: its row of
 * `gathered` is zero-filled and the handle remembers that it happened. */
int moe_regroup_gather(moe_sampler* sampler, void* stream, const float* hidden, uint32_t token_count, uint32_t columns,
                       const uint32_t* route_token, uint32_t route_count, float* gathered);
/* Synchronises `stream`, reports in *out_of_range whether any moe_regroup_gather
 * call on this handle since the last check met a token index >= token_count
 * (1) or not (0), and clears the mark.  No reference counterpart: the
 * reference indexes its host vector unchecked. */
int moe_regroup_gather_check(moe_sampler* sampler, void* stream, int32_t* out_of_range);

/* ---- latent-attention indexer ------------------------------------------- */

/* Replaces the selection at the end of select_compressed_indices
 * (src/kernels/cpu_latent_attention.cpp:414-423): std::partial_sort of the
 * {index, score} pairs with scored_index_precedes (:257-262: score descending,
 * index ascending on equal scores) and the first min(top_k, count) indices in
 * that order.  The scores themselves (:399-413) are the attention kernels'
 * business and are taken as input.
 *
 * scores      device, [rows x row_stride] fp32, count <= row_stride entries used per row
 * out_index   device, [rows x top_k]: the selected indices in rank order,
 *             0xFFFFFFFF in the slots beyond min(top_k, count)
 * out_score   device, [rows x top_k] or NULL: the scores of those indices
 * top_k <= MOE_INDEXER_TOPK_MAX.  NaN scores, for which the reference's order
 * is unspecified, rank last.  Asynchronous on `stream`; allocates nothing. */
#define MOE_INDEXER_TOPK_MAX 8192u
int moe_indexer_topk(moe_sampler* sampler, void* stream, const float* scores, uint32_t rows, uint32_t count, size_t row_stride,
                     uint32_t top_k, uint32_t* out_index, float* out_score);

#ifdef __cplusplus
}
#endif

#endif /* MOE_B200_SAMPLER_H */
