// TEST INFRASTRUCTURE ONLY.  This translation unit is the bridge between the
// parity tests and the *unmodified* reference sampler / expert dispatcher.
// It is compiled against the reference sources where they lie (never copied)
// by oracle/Makefile into oracle/_ref/libref_oracle.so.  Nothing in the
// shipped library links, loads or calls it.
//
// How it reaches the reference code:
//   * `#include "engine/session.cpp"` makes the file-static helpers of the
//     reference sampler visible here: LogitOrder (src/engine/session.cpp:26-36),
//     validate_sampling_options (:65-74) and sampling_distribution (:76-136).
//   * Session::sample (public API, include/ncnn/moe/session.h:326) is reached
//     through a Runtime with the reference's own FixtureModelAdapter
//     (tests/fixture_model_adapter.cpp) and a tiny on-disk fixture package.
//   * ExpertDispatcher::dispatch / dispatch_into
//     (include/ncnn/moe/expert_dispatcher.h:57-60) are called directly.
//
// The only logic restated here is the 10-line draw loop of
// Session::sample_unlocked (src/engine/session.cpp:429-442) so that an
// *injected* uniform can replace the Session's private mt19937_64, and the
// greedy scan (:404-424) which is unreachable without a Session.  Both are
// cross-checked against the public Session::sample by the CPU tests.

#include "engine/session.cpp" // NOLINT: deliberate TU inclusion, see above

#include "fixture_model_adapter.h"
#include "ncnn/moe/expert_dispatcher.h"
#include "ncnn/moe/runtime.h"

#include <atomic>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <memory>
#include <mutex>
#include <thread>
#include <unistd.h>

using namespace ncnn::moe;

namespace {

int status_of(const Error& error, char* message, size_t message_capacity)
{
    if (message != nullptr && message_capacity > 0)
    {
        std::snprintf(message, message_capacity, "%s", error.message.c_str());
    }
    return static_cast<int>(error.code) + 1;
}

void clear_message(char* message, size_t capacity)
{
    if (message != nullptr && capacity > 0)
        message[0] = '\0';
}

// Same control flow as Session::sample_unlocked(span, options) with the
// uniform supplied by the caller.  `used_uniform` reports whether the
// reference would have advanced its RNG.
int sample_injected(std::span<const float> logits, const SamplingOptions& options, float uniform,
                    int32_t* token, float* probability, int* used_uniform, char* message, size_t capacity)
{
    clear_message(message, capacity);
    if (used_uniform != nullptr)
        *used_uniform = 0;
    if (logits.empty())
        return status_of(Error{ErrorCode::InvalidArgument, "cannot sample empty logits"}, message, capacity);
    auto valid = validate_sampling_options(options);
    if (!valid)
        return status_of(valid.error(), message, capacity);
    if (options.temperature == 0.0f)
    {
        int32_t best = -1;
        float best_logit = -std::numeric_limits<float>::infinity();
        for (size_t index = 0; index < logits.size(); ++index)
        {
            const float logit = logits[index];
            if (!std::isfinite(logit))
                continue;
            if (best < 0 || logit > best_logit)
            {
                best = static_cast<int32_t>(index);
                best_logit = logit;
            }
        }
        if (best < 0)
            return status_of(Error{ErrorCode::InvalidArgument, "sampling requires at least one finite logit"}, message, capacity);
        *token = best;
        *probability = 1.0f;
        return 0;
    }
    auto candidates = sampling_distribution(logits, options);
    if (!candidates)
        return status_of(candidates.error(), message, capacity);
    const auto& list = candidates.value();
    if (list.size() == 1)
    {
        *token = list.front().token_id;
        *probability = 1.0f;
        return 0;
    }
    if (used_uniform != nullptr)
        *used_uniform = 1;
    float cumulative = 0.0f;
    for (const SamplingCandidate& candidate : list)
    {
        cumulative += candidate.probability;
        if (uniform < cumulative)
        {
            *token = candidate.token_id;
            *probability = candidate.probability;
            return 0;
        }
    }
    *token = list.back().token_id;
    *probability = list.back().probability;
    return 0;
}

inline float widen_bf16(uint16_t bits)
{
    const uint32_t wide = static_cast<uint32_t>(bits) << 16;
    float value;
    std::memcpy(&value, &wide, sizeof(value));
    return value;
}

class FixtureRuntime final : public Runtime
{
public:
    FixtureRuntime()
    {
        register_adapter(std::make_shared<FixtureModelAdapter>());
    }
};

struct FixtureWorld
{
    std::filesystem::path directory;
    std::unique_ptr<FixtureRuntime> runtime;
    ModelPtr model;
    std::string failure;

    FixtureWorld()
    {
        directory = std::filesystem::temp_directory_path() / ("b200_oracle_fixture_" + std::to_string(::getpid()));
        std::error_code ignored;
        std::filesystem::create_directories(directory, ignored);
        {
            // Manifest keys are the fixture adapter's input format
            // (tests/fixture_model_adapter.cpp); the values describe the
            // smallest model it accepts.
            std::ofstream manifest(directory / "config.json", std::ios::binary);
            manifest << "{\"model_type\":\"test_moe\",\"vocabulary_size\":4,\"hidden_size\":2,"
                        "\"intermediate_size\":2,\"layer_count\":1,\"expert_count\":2,"
                        "\"experts_per_token\":1,\"expert_activation\":\"relu\","
                        "\"expert_layout\":\"up_down\",\"normalize_topk_weights\":true,"
                        "\"use_expert_bias\":false,\"norm_epsilon\":0.00001,"
                        "\"weights_file\":\"model.test.bin\"}";
        }
        {
            // 40 floats; the sampler never looks at them.
            std::vector<float> weights(40);
            for (size_t index = 0; index < weights.size(); ++index)
                weights[index] = (index % 3 == 0) ? 1.0f : ((index % 3 == 1) ? 0.5f : -0.25f);
            std::ofstream file(directory / "model.test.bin", std::ios::binary);
            file.write(reinterpret_cast<const char*>(weights.data()), static_cast<std::streamsize>(weights.size() * sizeof(float)));
        }
        runtime = std::make_unique<FixtureRuntime>();
        RuntimeConfig config;
        config.hybrid_mode = HybridMode::CpuOnly;
        auto loaded = runtime->load_model(directory, config);
        if (!loaded)
        {
            failure = loaded.error().message;
            return;
        }
        model = loaded.value();
    }

    ~FixtureWorld()
    {
        model.reset();
        runtime.reset();
        std::error_code ignored;
        std::filesystem::remove_all(directory, ignored);
    }
};

FixtureWorld& world()
{
    static FixtureWorld instance;
    return instance;
}

struct SessionHandle
{
    SessionPtr session;
};

template<typename RowFunction>
void parallel_rows(size_t rows, int threads, RowFunction&& body)
{
    if (threads <= 1 || rows <= 1)
    {
        for (size_t row = 0; row < rows; ++row)
            body(row);
        return;
    }
    std::atomic<size_t> next{0};
    std::vector<std::thread> pool;
    const size_t count = std::min<size_t>(static_cast<size_t>(threads), rows);
    pool.reserve(count);
    for (size_t worker = 0; worker < count; ++worker)
    {
        pool.emplace_back([&]() {
            for (;;)
            {
                const size_t row = next.fetch_add(1);
                if (row >= rows)
                    return;
                body(row);
            }
        });
    }
    for (std::thread& thread : pool)
        thread.join();
}

} // namespace

extern "C" {

const char* oracle_kind()
{
    return "reference";
}

// sampling_distribution (src/engine/session.cpp:76-136): candidate ids and
// renormalised probabilities.  Returns 0 or ErrorCode+1.
int oracle_sampling_distribution(const float* logits, size_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                              int32_t* ids, float* probabilities, size_t capacity, size_t* count, char* message, size_t message_capacity)
{
    clear_message(message, message_capacity);
    SamplingOptions options{temperature, top_k, top_p, min_p};
    if (vocab == 0)
        return status_of(Error{ErrorCode::InvalidArgument, "cannot sample empty logits"}, message, message_capacity);
    auto valid = validate_sampling_options(options);
    if (!valid)
        return status_of(valid.error(), message, message_capacity);
    auto candidates = sampling_distribution(std::span<const float>(logits, vocab), options);
    if (!candidates)
        return status_of(candidates.error(), message, message_capacity);
    const auto& list = candidates.value();
    *count = list.size();
    for (size_t index = 0; index < list.size() && index < capacity; ++index)
    {
        ids[index] = list[index].token_id;
        probabilities[index] = list[index].probability;
    }
    return 0;
}

// The verification step of speculative decoding (src/engine/session.cpp:776-880)
// for one Session.  The reference's own sampling_distribution and
// candidate_probability do the work; restated here are only the accept loop
// around them and the draw of sample_residual_distribution (:150-202), so that
// injected uniforms can replace the Session's mt19937_64.  The residual
// restatement is cross-checked against the reference function itself by
// oracle_residual_with_generator below.
static int residual_injected(std::span<const SamplingCandidate> target, std::span<const SamplingCandidate> draft, size_t vocabulary_size,
                             float uniform, int32_t* token, float* probability, char* message, size_t capacity)
{
    std::vector<float> residual(vocabulary_size, 0.0f);
    for (const SamplingCandidate& candidate : target)
        residual[candidate.token_id] = candidate.probability;
    for (const SamplingCandidate& candidate : draft)
        residual[candidate.token_id] = std::max(0.0f, residual[candidate.token_id] - candidate.probability);
    const float normalizer = std::accumulate(residual.begin(), residual.end(), 0.0f);
    if (!std::isfinite(normalizer) || normalizer <= 0.0f)
        return status_of(Error{ErrorCode::InternalError, "speculative residual distribution is empty"}, message, capacity);
    const float sample_value = uniform * normalizer; // uniform_real_distribution<float>(0, normalizer): canonical * (b - a) + a
    float cumulative = 0.0f;
    for (size_t token_id = 0; token_id < residual.size(); ++token_id)
    {
        cumulative += residual[token_id];
        if (sample_value < cumulative)
        {
            *token = static_cast<int32_t>(token_id);
            *probability = residual[token_id] / normalizer;
            return 0;
        }
    }
    for (size_t token_id = residual.size(); token_id != 0; --token_id)
    {
        if (residual[token_id - 1] > 0.0f)
        {
            *token = static_cast<int32_t>(token_id - 1);
            *probability = residual[token_id - 1] / normalizer;
            return 0;
        }
    }
    return status_of(Error{ErrorCode::InternalError, "speculative residual sampling failed"}, message, capacity);
}

int oracle_speculative_verify(const float* target_logits, const float* draft_logits, size_t vocab, size_t draft_count, const int32_t* proposed,
                              float temperature, uint32_t top_k, float top_p, float min_p, const float* uniforms, uint32_t* accepted_out,
                              float* accepted_probability, int32_t* next_token, float* next_probability, uint32_t* uniforms_used, char* message,
                              size_t capacity)
{
    clear_message(message, capacity);
    const SamplingOptions options{temperature, top_k, top_p, min_p};
    size_t used = 0;
    size_t accepted = 0;
    std::vector<SamplingCandidate> rejected_target, rejected_draft;
    *uniforms_used = 0;
    *accepted_out = 0;
    while (accepted < draft_count)
    {
        const std::span<const float> target_row(target_logits + accepted * vocab, vocab);
        if (temperature == 0.0f)
        {
            int32_t token = -1;
            float probability = 0.0f;
            if (int status = sample_injected(target_row, options, 0.0f, &token, &probability, nullptr, message, capacity))
                return status;
            if (token != proposed[accepted])
                break;
            accepted_probability[accepted] = 1.0f;
        }
        else
        {
            auto valid = validate_sampling_options(options);
            if (!valid)
                return status_of(valid.error(), message, capacity);
            auto target_distribution = sampling_distribution(target_row, options);
            auto draft_distribution = sampling_distribution(std::span<const float>(draft_logits + accepted * vocab, vocab), options);
            if (!target_distribution || !draft_distribution)
                return status_of(!target_distribution ? target_distribution.error() : draft_distribution.error(), message, capacity);
            const float target_probability = candidate_probability(target_distribution.value(), proposed[accepted]);
            const float draft_probability = candidate_probability(draft_distribution.value(), proposed[accepted]);
            if (draft_probability <= 0.0f)
                return status_of(Error{ErrorCode::InternalError, "sampled draft token has zero probability"}, message, capacity);
            const float acceptance_probability = std::min(1.0f, target_probability / draft_probability);
            if (uniforms[used++] >= acceptance_probability)
            {
                rejected_target = std::move(target_distribution).value();
                rejected_draft = std::move(draft_distribution).value();
                break;
            }
            accepted_probability[accepted] = target_probability;
        }
        ++accepted;
    }
    int status = 0;
    if (accepted < draft_count && temperature > 0.0f)
    {
        status = residual_injected(rejected_target, rejected_draft, vocab, uniforms[used++], next_token, next_probability, message, capacity);
    }
    else
    {
        int used_uniform = 0;
        status = sample_injected(std::span<const float>(target_logits + accepted * vocab, vocab), options, uniforms[used], next_token,
                                 next_probability, &used_uniform, message, capacity);
        used += static_cast<size_t>(used_uniform);
    }
    *accepted_out = static_cast<uint32_t>(accepted);
    *uniforms_used = static_cast<uint32_t>(used);
    return status;
}

// The reference's sample_residual_distribution itself, driven by a fresh
// std::mt19937_64(seed) exactly as a Session would, on the distributions of
// two logit rows.  Pins residual_injected: oracle_mt19937_uniforms(seed, 1)
// gives the uniform this call consumes.
int oracle_residual_with_generator(const float* target_logits, const float* draft_logits, size_t vocab, float temperature, uint32_t top_k,
                                   float top_p, float min_p, uint64_t seed, int32_t* token, float* probability, char* message, size_t capacity)
{
    clear_message(message, capacity);
    const SamplingOptions options{temperature, top_k, top_p, min_p};
    auto target_distribution = sampling_distribution(std::span<const float>(target_logits, vocab), options);
    auto draft_distribution = sampling_distribution(std::span<const float>(draft_logits, vocab), options);
    if (!target_distribution || !draft_distribution)
        return status_of(!target_distribution ? target_distribution.error() : draft_distribution.error(), message, capacity);
    std::mt19937_64 generator(seed);
    auto sampled = sample_residual_distribution(target_distribution.value(), draft_distribution.value(), vocab, generator);
    if (!sampled)
        return status_of(sampled.error(), message, capacity);
    *token = sampled.value().token_id;
    *probability = sampled.value().probability;
    return 0;
}

int oracle_sample_with_uniform(const float* logits, size_t vocab, float temperature, uint32_t top_k, float top_p, float min_p, float uniform,
                            int32_t* token, float* probability, int* used_uniform, char* message, size_t message_capacity)
{
    return sample_injected(std::span<const float>(logits, vocab), SamplingOptions{temperature, top_k, top_p, min_p}, uniform,
                           token, probability, used_uniform, message, message_capacity);
}

// First `count` entries of std::stable_sort(ids, LogitOrder{logits})
// (src/engine/session.cpp:80-82) = the Top-K index set, in rank order.
void oracle_topk_order(const float* logits, size_t vocab, size_t count, int32_t* ids)
{
    std::vector<int32_t> order(vocab);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), LogitOrder{std::span<const float>(logits, vocab)});
    for (size_t index = 0; index < count && index < vocab; ++index)
        ids[index] = order[index];
}

// Batched form used for parity at scale and for the timed CPU baseline:
// every row is one independent call of the sampler with its own options and
// its own injected uniform.  dtype 0 = fp32, 1 = bf16 (widened exactly,
// src/kernels/cpu_bfloat16.cpp:26-28 is the reference's own widening).
int oracle_sample_batch(const void* logits, int dtype, size_t rows, size_t vocab, size_t row_stride,
                     const float* temperature, const uint32_t* top_k, const float* top_p, const float* min_p,
                     const float* uniforms, int32_t* tokens, float* probabilities, int32_t* statuses, int32_t* used_uniform, int threads)
{
    parallel_rows(rows, threads, [&](size_t row) {
        std::vector<float> widened;
        const float* values = nullptr;
        if (dtype == 0)
        {
            values = static_cast<const float*>(logits) + row * row_stride;
        }
        else
        {
            const uint16_t* source = static_cast<const uint16_t*>(logits) + row * row_stride;
            widened.resize(vocab);
            for (size_t index = 0; index < vocab; ++index)
                widened[index] = widen_bf16(source[index]);
            values = widened.data();
        }
        int32_t token = -1;
        float probability = 0.0f;
        int used = 0;
        const int status = sample_injected(std::span<const float>(values, vocab),
                                           SamplingOptions{temperature[row], top_k[row], top_p[row], min_p[row]},
                                           uniforms[row], &token, &probability, &used, nullptr, 0);
        tokens[row] = token;
        probabilities[row] = probability;
        statuses[row] = status;
        if (used_uniform != nullptr)
            used_uniform[row] = used;
    });
    return 0;
}

// Public-API route: Runtime + fixture model + Session::sample, the Session's
// own mt19937_64 seeded with `seed` (src/engine/session.cpp:291).
void* oracle_session_create(uint64_t seed, char* message, size_t message_capacity)
{
    clear_message(message, message_capacity);
    FixtureWorld& fixture = world();
    if (!fixture.model)
    {
        if (message != nullptr && message_capacity > 0)
            std::snprintf(message, message_capacity, "fixture model failed to load: %s", fixture.failure.c_str());
        return nullptr;
    }
    SessionOptions options;
    options.sampling_seed = seed;
    auto session = fixture.runtime->create_session(fixture.model, options);
    if (!session)
    {
        status_of(session.error(), message, message_capacity);
        return nullptr;
    }
    return new SessionHandle{session.value()};
}

int oracle_session_sample(void* handle, const float* logits, size_t vocab, float temperature, uint32_t top_k, float top_p, float min_p,
                       int32_t* token, float* probability, char* message, size_t message_capacity)
{
    clear_message(message, message_capacity);
    LogitsOutput output;
    output.values.assign(logits, logits + vocab);
    auto sampled = static_cast<SessionHandle*>(handle)->session->sample(output, SamplingOptions{temperature, top_k, top_p, min_p});
    if (!sampled)
        return status_of(sampled.error(), message, message_capacity);
    *token = sampled.value().token_id;
    *probability = sampled.value().probability;
    return 0;
}

void oracle_session_destroy(void* handle)
{
    delete static_cast<SessionHandle*>(handle);
}

// The uniform a Session would draw: std::uniform_real_distribution<float>(0,1)
// over std::mt19937_64 (src/engine/session.cpp:432-433), `count` draws.
void oracle_mt19937_uniforms(uint64_t seed, size_t count, float* values)
{
    std::mt19937_64 generator(seed);
    std::uniform_real_distribution<float> distribution(0.0f, 1.0f);
    for (size_t index = 0; index < count; ++index)
        values[index] = distribution(generator);
}

// ExpertDispatcher::dispatch / dispatch_into flattened to CSR arrays.
// score_function: 0 Softmax, 1 Sigmoid, 2 SqrtSoftplus; normalization: 0 None,
// 1 SelectedExperts.  Outputs: batch_expert[batch_count],
// batch_offset[batch_count+1], and per route token/rank/weight.
int oracle_expert_dispatch(int use_dispatch_into, const float* router_logits, size_t logit_count, uint32_t token_count,
                        uint32_t expert_count, uint32_t top_k, int score_function, int normalization, float scaling,
                        const float* selection_bias, size_t bias_count, const uint32_t* explicit_ids, size_t explicit_count, uint32_t flags,
                        uint32_t* batch_expert, uint32_t* batch_offset, uint32_t* route_token, uint32_t* route_rank, float* route_weight,
                        size_t route_capacity, size_t* batch_count, size_t* assignment_count, char* message, size_t message_capacity)
{
    clear_message(message, message_capacity);
    ExpertDispatchOptions options;
    options.expert_count = expert_count;
    options.top_k = top_k;
    options.score_function = static_cast<RouterScoreFunction>(score_function);
    options.normalization = static_cast<RouterNormalization>(normalization);
    options.routed_scaling_factor = scaling;
    if (selection_bias != nullptr)
        options.selection_bias = std::span<const float>(selection_bias, bias_count);
    if (explicit_ids != nullptr)
        options.explicit_expert_ids = std::span<const uint32_t>(explicit_ids, explicit_count);
    options.flags = flags;
    ExpertDispatcher dispatcher;
    ExpertDispatchPlan plan;
    const std::span<const float> logits(router_logits, logit_count);
    if (use_dispatch_into != 0)
    {
        auto status = dispatcher.dispatch_into(logits, token_count, options, plan);
        if (!status)
            return status_of(status.error(), message, message_capacity);
    }
    else
    {
        auto dispatched = dispatcher.dispatch(logits, token_count, options);
        if (!dispatched)
            return status_of(dispatched.error(), message, message_capacity);
        plan = std::move(dispatched).value();
    }
    *batch_count = plan.batches.size();
    *assignment_count = plan.assignment_count;
    size_t cursor = 0;
    for (size_t batch = 0; batch < plan.batches.size(); ++batch)
    {
        batch_expert[batch] = plan.batches[batch].expert_id;
        batch_offset[batch] = static_cast<uint32_t>(cursor);
        for (const ExpertRoute& route : plan.batches[batch].routes)
        {
            if (cursor < route_capacity)
            {
                route_token[cursor] = route.token_index;
                route_rank[cursor] = route.rank;
                route_weight[cursor] = route.weight;
            }
            ++cursor;
        }
    }
    batch_offset[plan.batches.size()] = static_cast<uint32_t>(cursor);
    return 0;
}

} // extern "C"
