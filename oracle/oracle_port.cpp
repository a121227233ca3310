// TEST INFRASTRUCTURE ONLY.  A CPU restatement of the reference's generation
// sampler and expert dispatcher, written from the behaviour of
//   src/engine/session.cpp:26-36,65-136,393-443   (sampler)
//   src/graph/expert_dispatcher.cpp:19-158        (router scoring, Top-K, grouping)
// It is the parity checker for the CUDA path on machines where the reference
// checkout is absent; it is pinned against the reference itself (built as
// oracle/_ref/libref_oracle.so) and against the committed golden vectors by
// the CPU tests.  The shipped library never links, loads or calls this file.
//
// Two exponential modes are offered (oracle_set_exp_mode):
//   0  libm expf / log1pf — what the reference executes;
//   1  double-precision exp / log1p rounded once to float — what the device
//      code executes.  Mode 1 differs from mode 0 by one ulp for roughly
//      6e-4 of arguments; it exists so that every other arithmetic step of a
//      kernel can be checked bit for bit.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <numeric>
#include <thread>
#include <vector>

namespace {

std::atomic<int> g_exp_mode{0};

enum Status : int
{
    kOk = 0,
    kInvalidArgument = 1, // ErrorCode::InvalidArgument + 1 (include/ncnn/moe/result.h:12-19)
    kInvalidModel = 3,    // ErrorCode::InvalidModel + 1
    kInternalError = 5,   // ErrorCode::InternalError + 1
};

inline float exp_f(float x)
{
    if (g_exp_mode.load(std::memory_order_relaxed) == 0)
        return std::exp(x);
    return static_cast<float>(std::exp(static_cast<double>(x)));
}

inline float log1p_f(float x)
{
    if (g_exp_mode.load(std::memory_order_relaxed) == 0)
        return std::log1p(x);
    return static_cast<float>(std::log1p(static_cast<double>(x)));
}

int fail(int status, const char* text, char* message, size_t capacity)
{
    if (message != nullptr && capacity > 0)
        std::snprintf(message, capacity, "%s", text);
    return status;
}

struct Options
{
    float temperature;
    uint32_t top_k;
    float top_p;
    float min_p;
};

struct Candidate
{
    int32_t id;
    float p;
};

// session.cpp:65-74 — the three range checks and their messages.
int check_options(const Options& o, char* message, size_t capacity)
{
    if (!std::isfinite(o.temperature) || o.temperature < 0.0f)
        return fail(kInvalidArgument, "temperature must be finite and non-negative", message, capacity);
    if (!std::isfinite(o.top_p) || o.top_p <= 0.0f || o.top_p > 1.0f)
        return fail(kInvalidArgument, "top_p must be in the range (0, 1]", message, capacity);
    if (!std::isfinite(o.min_p) || o.min_p < 0.0f || o.min_p > 1.0f)
        return fail(kInvalidArgument, "min_p must be in the range [0, 1]", message, capacity);
    return kOk;
}

// Rank order of session.cpp:26-36,80-82: logit descending, index ascending on
// equal values (so -0.0 and +0.0 tie).  NaN makes the reference comparator
// inconsistent (its result is unspecified); here NaN ranks after everything,
// which is also what the device code does.
void rank_order(const float* logits, size_t vocab, std::vector<int32_t>& order)
{
    order.resize(vocab);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [logits](int32_t a, int32_t b) {
        const float x = logits[a];
        const float y = logits[b];
        const bool x_nan = x != x;
        const bool y_nan = y != y;
        if (x_nan || y_nan)
            return !x_nan && y_nan;
        return x > y;
    });
}

// session.cpp:76-136.  Every sum is a left-to-right fp32 accumulation in rank
// order; Top-K, then Min-P, then Top-P; renormalise at the end.
int distribution(const float* logits, size_t vocab, const Options& o, std::vector<Candidate>& kept, char* message, size_t capacity)
{
    std::vector<int32_t> order;
    rank_order(logits, vocab, order);
    if (!std::isfinite(logits[order[0]]))
        return fail(kInvalidArgument, "sampling requires at least one finite logit", message, capacity);
    size_t considered = vocab;
    if (o.top_k > 0 && o.top_k < vocab)
        considered = o.top_k;

    const float peak = logits[order[0]] / o.temperature;
    kept.clear();
    kept.reserve(considered);
    float total = 0.0f;
    for (size_t rank = 0; rank < considered; ++rank)
    {
        const float value = logits[order[rank]];
        if (!std::isfinite(value))
            continue;
        const float weight = exp_f(value / o.temperature - peak);
        kept.push_back({order[rank], weight});
        total += weight;
    }
    if (kept.empty() || !std::isfinite(total) || total <= 0.0f)
        return fail(kInvalidArgument, "sampling distribution is invalid", message, capacity);
    for (Candidate& c : kept)
        c.p /= total;

    if (o.min_p > 0.0f)
    {
        const float floor_p = kept[0].p * o.min_p;
        size_t write = 0;
        for (size_t read = 0; read < kept.size(); ++read)
            if (kept[read].p >= floor_p)
                kept[write++] = kept[read];
        kept.resize(write);
    }

    float running = 0.0f;
    size_t nucleus = 0;
    while (nucleus < kept.size())
    {
        running += kept[nucleus].p;
        ++nucleus;
        if (running >= o.top_p)
            break;
    }
    kept.resize(nucleus);

    total = 0.0f;
    for (const Candidate& c : kept)
        total += c.p;
    for (Candidate& c : kept)
        c.p /= total;
    return kOk;
}

// session.cpp:393-443 with the uniform supplied by the caller.
int sample_one(const float* logits, size_t vocab, const Options& o, float uniform, int32_t* token, float* probability, int* used_uniform,
               char* message, size_t capacity)
{
    if (message != nullptr && capacity > 0)
        message[0] = '\0';
    if (used_uniform != nullptr)
        *used_uniform = 0;
    if (vocab == 0)
        return fail(kInvalidArgument, "cannot sample empty logits", message, capacity);
    if (int status = check_options(o, message, capacity))
        return status;
    if (o.temperature == 0.0f)
    {
        // greedy: first index of the largest finite logit (:404-424)
        int64_t best = -1;
        for (size_t index = 0; index < vocab; ++index)
        {
            if (!std::isfinite(logits[index]))
                continue;
            if (best < 0 || logits[index] > logits[best])
                best = static_cast<int64_t>(index);
        }
        if (best < 0)
            return fail(kInvalidArgument, "sampling requires at least one finite logit", message, capacity);
        *token = static_cast<int32_t>(best);
        *probability = 1.0f;
        return kOk;
    }
    std::vector<Candidate> kept;
    if (int status = distribution(logits, vocab, o, kept, message, capacity))
        return status;
    if (kept.size() == 1)
    {
        *token = kept[0].id;
        *probability = 1.0f;
        return kOk;
    }
    if (used_uniform != nullptr)
        *used_uniform = 1;
    float running = 0.0f;
    for (const Candidate& c : kept)
    {
        running += c.p;
        if (uniform < running)
        {
            *token = c.id;
            *probability = c.p;
            return kOk;
        }
    }
    *token = kept.back().id;
    *probability = kept.back().p;
    return kOk;
}

// candidate_probability (session.cpp:138-148).
float probability_of(const std::vector<Candidate>& list, int32_t token)
{
    for (const Candidate& c : list)
        if (c.id == token)
            return c.p;
    return 0.0f;
}

// sample_residual_distribution (session.cpp:150-202) with the uniform supplied
// by the caller: residual = max(0, target - draft) per token id, summed in
// token-id order; the draw is uniform * normaliser.
int residual_sample(const std::vector<Candidate>& target, const std::vector<Candidate>& draft, size_t vocab, float uniform, int32_t* token,
                    float* probability, char* message, size_t capacity)
{
    std::vector<float> residual(vocab, 0.0f);
    for (const Candidate& c : target)
        residual[static_cast<size_t>(c.id)] = c.p;
    for (const Candidate& c : draft)
    {
        float& slot = residual[static_cast<size_t>(c.id)];
        const float reduced = slot - c.p;
        slot = reduced > 0.0f ? reduced : 0.0f;
    }
    float normaliser = 0.0f;
    for (float value : residual)
        normaliser += value;
    if (!std::isfinite(normaliser) || normaliser <= 0.0f)
        return fail(kInternalError, "speculative residual distribution is empty", message, capacity);
    const float sample_value = uniform * normaliser;
    float running = 0.0f;
    for (size_t id = 0; id < vocab; ++id)
    {
        running += residual[id];
        if (sample_value < running)
        {
            *token = static_cast<int32_t>(id);
            *probability = residual[id] / normaliser;
            return kOk;
        }
    }
    for (size_t id = vocab; id != 0; --id)
    {
        if (residual[id - 1] > 0.0f)
        {
            *token = static_cast<int32_t>(id - 1);
            *probability = residual[id - 1] / normaliser;
            return kOk;
        }
    }
    return fail(kInternalError, "speculative residual sampling failed", message, capacity);
}

inline float widen_bf16(uint16_t bits)
{
    const uint32_t wide = static_cast<uint32_t>(bits) << 16;
    float value;
    std::memcpy(&value, &wide, sizeof(value));
    return value;
}

template<typename Body>
void for_rows(size_t rows, int threads, Body&& body)
{
    if (threads <= 1 || rows <= 1)
    {
        for (size_t row = 0; row < rows; ++row)
            body(row);
        return;
    }
    std::atomic<size_t> cursor{0};
    const size_t workers = std::min<size_t>(static_cast<size_t>(threads), rows);
    std::vector<std::thread> pool;
    for (size_t w = 0; w < workers; ++w)
        pool.emplace_back([&]() {
            for (size_t row = cursor.fetch_add(1); row < rows; row = cursor.fetch_add(1))
                body(row);
        });
    for (auto& t : pool)
        t.join();
}

// ---- Philox4x32-10 (Salmon, Moraes, Dror, Shaw, SC'11) -----------------------
// The harness convention: key = (seed lo, seed hi), counter = (row lo, row hi,
// step lo, step hi); the uniform is the top 24 bits of output word 0 scaled by
// 2^-24, so it lies in [0, 1) and is exactly representable.
inline void philox_round(uint32_t (&c)[4], const uint32_t (&k)[2])
{
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c[0];
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c[2];
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k[0];
    const uint32_t n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k[1];
    const uint32_t n3 = static_cast<uint32_t>(p0);
    c[0] = n0;
    c[1] = n1;
    c[2] = n2;
    c[3] = n3;
}

void philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4])
{
    uint32_t c[4] = {counter[0], counter[1], counter[2], counter[3]};
    uint32_t k[2] = {key[0], key[1]};
    for (int round = 0; round < 10; ++round)
    {
        philox_round(c, k);
        k[0] += 0x9E3779B9u;
        k[1] += 0xBB67AE85u;
    }
    for (int i = 0; i < 4; ++i)
        out[i] = c[i];
}

// ---- router ------------------------------------------------------------------

// expert_dispatcher.cpp:24-59
float softplus_f(float x)
{
    if (x > 20.0f)
        return x;
    if (x < -20.0f)
        return exp_f(x);
    return log1p_f(exp_f(x));
}

void token_scores(const float* logits, uint32_t experts, int score_function, std::vector<float>& scores)
{
    scores.resize(experts);
    if (score_function == 0)
    {
        float peak = logits[0];
        for (uint32_t e = 1; e < experts; ++e)
            peak = std::max(peak, logits[e]);
        float total = 0.0f;
        for (uint32_t e = 0; e < experts; ++e)
        {
            scores[e] = exp_f(logits[e] - peak);
            total += scores[e];
        }
        for (uint32_t e = 0; e < experts; ++e)
            scores[e] /= total;
        return;
    }
    for (uint32_t e = 0; e < experts; ++e)
    {
        if (score_function == 1)
            scores[e] = 1.0f / (1.0f + exp_f(-logits[e]));
        else
            scores[e] = std::sqrt(softplus_f(logits[e]));
    }
}

struct Pick
{
    uint32_t expert;
    float key;
};

} // namespace

extern "C" {

const char* oracle_kind()
{
    return "port";
}

void oracle_set_exp_mode(int mode)
{
    g_exp_mode.store(mode);
}

int oracle_sampling_distribution(const float* logits, size_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                                 int32_t* ids, float* probabilities, size_t capacity, size_t* count, char* message, size_t message_capacity)
{
    if (message != nullptr && message_capacity > 0)
        message[0] = '\0';
    const Options o{temperature, top_k, top_p, min_p};
    if (vocab == 0)
        return fail(kInvalidArgument, "cannot sample empty logits", message, message_capacity);
    if (int status = check_options(o, message, message_capacity))
        return status;
    std::vector<Candidate> kept;
    if (int status = distribution(logits, vocab, o, kept, message, message_capacity))
        return status;
    *count = kept.size();
    for (size_t i = 0; i < kept.size() && i < capacity; ++i)
    {
        ids[i] = kept[i].id;
        probabilities[i] = kept[i].p;
    }
    return kOk;
}

int oracle_sample_with_uniform(const float* logits, size_t vocab, float temperature, uint32_t top_k, float top_p, float min_p, float uniform,
                               int32_t* token, float* probability, int* used_uniform, char* message, size_t message_capacity)
{
    return sample_one(logits, vocab, Options{temperature, top_k, top_p, min_p}, uniform, token, probability, used_uniform, message, message_capacity);
}

void oracle_topk_order(const float* logits, size_t vocab, size_t count, int32_t* ids)
{
    std::vector<int32_t> order;
    rank_order(logits, vocab, order);
    for (size_t i = 0; i < count && i < vocab; ++i)
        ids[i] = order[i];
}

int oracle_sample_batch(const void* logits, int dtype, size_t rows, size_t vocab, size_t row_stride,
                        const float* temperature, const uint32_t* top_k, const float* top_p, const float* min_p,
                        const float* uniforms, int32_t* tokens, float* probabilities, int32_t* statuses, int32_t* used_uniform, int threads)
{
    for_rows(rows, threads, [&](size_t row) {
        std::vector<float> widened;
        const float* values;
        if (dtype == 0)
        {
            values = static_cast<const float*>(logits) + row * row_stride;
        }
        else
        {
            const uint16_t* source = static_cast<const uint16_t*>(logits) + row * row_stride;
            widened.resize(vocab);
            for (size_t i = 0; i < vocab; ++i)
                widened[i] = widen_bf16(source[i]);
            values = widened.data();
        }
        int32_t token = -1;
        float probability = 0.0f;
        int used = 0;
        statuses[row] = sample_one(values, vocab, Options{temperature[row], top_k[row], top_p[row], min_p[row]}, uniforms[row],
                                   &token, &probability, &used, nullptr, 0);
        tokens[row] = token;
        probabilities[row] = probability;
        if (used_uniform != nullptr)
            used_uniform[row] = used;
    });
    return kOk;
}

// The verification step of speculative decoding (session.cpp:776-880) for one
// Session: `proposed[0..draft_count)` against target_logits[(draft_count + 1) x vocab]
// and draft_logits[draft_count x vocab]; uniforms are consumed in order.
int oracle_speculative_verify(const float* target_logits, const float* draft_logits, size_t vocab, size_t draft_count, const int32_t* proposed,
                              float temperature, uint32_t top_k, float top_p, float min_p, const float* uniforms, uint32_t* accepted_out,
                              float* accepted_probability, int32_t* next_token, float* next_probability, uint32_t* uniforms_used, char* message,
                              size_t capacity)
{
    const Options o{temperature, top_k, top_p, min_p};
    if (message != nullptr && capacity > 0)
        message[0] = '\0';
    size_t used = 0;
    size_t accepted = 0;
    std::vector<Candidate> rejected_target, rejected_draft;
    *uniforms_used = 0;
    *accepted_out = 0;
    while (accepted < draft_count)
    {
        const float* target_row = target_logits + accepted * vocab;
        if (temperature == 0.0f)
        {
            int32_t token = -1;
            float probability = 0.0f;
            if (int status = sample_one(target_row, vocab, o, 0.0f, &token, &probability, nullptr, message, capacity))
                return status;
            if (token != proposed[accepted])
                break;
            accepted_probability[accepted] = 1.0f;
        }
        else
        {
            if (vocab == 0)
                return fail(kInvalidArgument, "cannot sample empty logits", message, capacity);
            if (int status = check_options(o, message, capacity))
                return status;
            std::vector<Candidate> target, draft;
            if (int status = distribution(target_row, vocab, o, target, message, capacity))
                return status;
            if (int status = distribution(draft_logits + accepted * vocab, vocab, o, draft, message, capacity))
                return status;
            const float target_probability = probability_of(target, proposed[accepted]);
            const float draft_probability = probability_of(draft, proposed[accepted]);
            if (draft_probability <= 0.0f)
                return fail(kInternalError, "sampled draft token has zero probability", message, capacity);
            const float ratio = target_probability / draft_probability;
            const float acceptance = ratio < 1.0f ? ratio : 1.0f; // std::min(1.0f, ratio)
            if (uniforms[used++] >= acceptance)
            {
                rejected_target = std::move(target);
                rejected_draft = std::move(draft);
                break;
            }
            accepted_probability[accepted] = target_probability;
        }
        ++accepted;
    }
    int status = kOk;
    if (accepted < draft_count && temperature > 0.0f)
    {
        status = residual_sample(rejected_target, rejected_draft, vocab, uniforms[used++], next_token, next_probability, message, capacity);
    }
    else
    {
        int used_uniform = 0;
        status = sample_one(target_logits + accepted * vocab, vocab, o, uniforms[used], next_token, next_probability, &used_uniform, message, capacity);
        used += static_cast<size_t>(used_uniform);
    }
    *accepted_out = static_cast<uint32_t>(accepted);
    *uniforms_used = static_cast<uint32_t>(used);
    return status;
}

void oracle_philox4x32_10(const uint32_t* counter, const uint32_t* key, uint32_t* out)
{
    philox4x32_10(counter, key, out);
}

float oracle_philox_uniform(uint64_t seed, uint64_t row, uint64_t step)
{
    const uint32_t counter[4] = {static_cast<uint32_t>(row), static_cast<uint32_t>(row >> 32), static_cast<uint32_t>(step), static_cast<uint32_t>(step >> 32)};
    const uint32_t key[2] = {static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)};
    uint32_t out[4];
    philox4x32_10(counter, key, out);
    return static_cast<float>(out[0] >> 8) * 0x1.0p-24f;
}

// expert_dispatcher.cpp:79-158, flattened to CSR arrays (see ref_shim.cpp for
// the layout).  Validation order and messages follow the reference.
int oracle_expert_dispatch(int /*use_dispatch_into*/, const float* router_logits, size_t logit_count, uint32_t token_count,
                           uint32_t expert_count, uint32_t top_k, int score_function, int normalization, float scaling,
                           const float* selection_bias, size_t bias_count, const uint32_t* explicit_ids, size_t explicit_count, uint32_t flags,
                           uint32_t* batch_expert, uint32_t* batch_offset, uint32_t* route_token, uint32_t* route_rank, float* route_weight,
                           size_t route_capacity, size_t* batch_count, size_t* assignment_count, char* message, size_t message_capacity)
{
    if (message != nullptr && message_capacity > 0)
        message[0] = '\0';
    if (token_count == 0)
        return fail(kInvalidArgument, "expert dispatch requires at least one token", message, message_capacity);
    if (expert_count == 0 || top_k == 0 || top_k > expert_count)
        return fail(kInvalidArgument, "expert dispatch requires 0 < top_k <= expert_count", message, message_capacity);
    if (logit_count / expert_count != token_count || logit_count % expert_count != 0)
        return fail(kInvalidArgument, "router logits shape does not match token and expert counts", message, message_capacity);
    if (selection_bias != nullptr && bias_count != 0 && bias_count != expert_count)
        return fail(kInvalidArgument, "router selection bias must match expert_count", message, message_capacity);
    if (explicit_ids != nullptr && explicit_count != 0 && explicit_count != static_cast<size_t>(token_count) * top_k)
        return fail(kInvalidArgument, "explicit expert ids must match token_count * top_k", message, message_capacity);
    if (!std::isfinite(scaling) || scaling <= 0.0f)
        return fail(kInvalidArgument, "routed scaling factor must be finite and positive", message, message_capacity);
    for (size_t i = 0; i < logit_count; ++i)
        if (!std::isfinite(router_logits[i]))
            return fail(kInvalidArgument, "router logits must be finite", message, message_capacity);

    const bool has_bias = selection_bias != nullptr && bias_count != 0;
    const bool has_explicit = explicit_ids != nullptr && explicit_count != 0;
    const bool renormalize = (flags & 1u) != 0 || normalization == 1;

    struct Route
    {
        uint32_t token, rank;
        float weight;
    };
    std::vector<std::vector<Route>> per_expert(expert_count);
    std::vector<float> scores;
    std::vector<Pick> picks;
    for (uint32_t token = 0; token < token_count; ++token)
    {
        token_scores(router_logits + static_cast<size_t>(token) * expert_count, expert_count, score_function, scores);
        picks.clear();
        if (has_explicit)
        {
            for (uint32_t r = 0; r < top_k; ++r)
            {
                const uint32_t expert = explicit_ids[static_cast<size_t>(token) * top_k + r];
                if (expert >= expert_count)
                    return fail(kInvalidArgument, "explicit expert id is out of range", message, message_capacity);
                picks.push_back({expert, scores[expert]});
            }
        }
        else
        {
            // stable Top-K: key descending, expert id ascending (:19-22,61-77)
            std::vector<Pick> all(expert_count);
            for (uint32_t e = 0; e < expert_count; ++e)
                all[e] = {e, scores[e] + (has_bias ? selection_bias[e] : 0.0f)};
            std::stable_sort(all.begin(), all.end(), [](const Pick& a, const Pick& b) { return a.key > b.key; });
            picks.assign(all.begin(), all.begin() + top_k);
        }
        float chosen_total = 0.0f;
        for (const Pick& p : picks)
            chosen_total += scores[p.expert];
        if (renormalize && chosen_total <= 0.0f)
            return fail(kInvalidModel, "selected router weights have a non-positive sum", message, message_capacity);
        for (uint32_t rank = 0; rank < picks.size(); ++rank)
        {
            const float s = scores[picks[rank].expert];
            const float weight = (renormalize ? s / chosen_total : s) * scaling;
            per_expert[picks[rank].expert].push_back({token, rank, weight});
        }
    }
    size_t batches = 0;
    size_t cursor = 0;
    for (uint32_t e = 0; e < expert_count; ++e)
    {
        if (per_expert[e].empty())
            continue;
        batch_expert[batches] = e;
        batch_offset[batches] = static_cast<uint32_t>(cursor);
        for (const Route& r : per_expert[e])
        {
            if (cursor < route_capacity)
            {
                route_token[cursor] = r.token;
                route_rank[cursor] = r.rank;
                route_weight[cursor] = r.weight;
            }
            ++cursor;
        }
        ++batches;
    }
    batch_offset[batches] = static_cast<uint32_t>(cursor);
    *batch_count = batches;
    *assignment_count = static_cast<size_t>(token_count) * top_k;
    return kOk;
}

// The selection of src/kernels/cpu_latent_attention.cpp:414-423: {index, score}
// pairs ordered by scored_index_precedes (:257-262) with std::partial_sort, the
// first min(top_k, count) indices returned.  (The reference function is a
// file-static of that translation unit; the statement here is line for line.)
void oracle_indexer_topk(const float* scores, size_t count, size_t top_k, uint32_t* selected_indices)
{
    struct ScoredIndex
    {
        uint32_t index;
        float score;
    };
    std::vector<ScoredIndex> scored(count);
    for (uint32_t index = 0; index < count; ++index)
        scored[index] = {index, scores[index]};
    const size_t selected_count = std::min(top_k, count);
    std::partial_sort(scored.begin(), scored.begin() + selected_count, scored.end(), [](const ScoredIndex& left, const ScoredIndex& right) {
        return left.score > right.score || (left.score == right.score && left.index < right.index);
    });
    for (size_t index = 0; index < selected_count; ++index)
        selected_indices[index] = scored[index].index;
}

} // extern "C"
