// C++20 host adapter over the C ABI (include/moe_b200_sampler.h).
//
// It gives callers of the reference runtime the same shapes they already use —
// SamplingOptions / SampledToken (include/ncnn/moe/session.h:49-61),
// Result<T> / Error / ErrorCode (include/ncnn/moe/result.h:12-97),
// ExpertDispatchOptions / ExpertDispatchPlan / ExpertRoute / ExpertBatch
// (include/ncnn/moe/expert_dispatcher.h:15-51) — with the work done on the GPU:
//
//   DeviceSampler::sample          stands in for Session::sample            (session.h:326)
//   DeviceSampler::sample_batch    stands in for the per-Session loop of    examples/internal/run_model.cpp:776-809
//   DeviceSampler::verify_speculative   for the verification step of        src/engine/session.cpp:776-880
//   DeviceExpertDispatcher::dispatch / dispatch_into   for ExpertDispatcher (expert_dispatcher.h:57-60)
//
// Errors are values, never exceptions, and carry the reference's messages.
// The one deliberate difference: a Session draws from a private
// std::mt19937_64; here every draw is Philox4x32-10 of (seed, row id, step), so
// a row's uniform does not depend on how many other rows consumed one.
//
// Header-only; link against libmoe_b200_sampler.so.
#pragma once

#include <cstdint>
#include <memory>
#include <span>
#include <string>
#include <utility>
#include <variant>
#include <vector>

#include "../../include/moe_b200_sampler.h"

namespace moe_b200 {

enum class ErrorCode
{
    InvalidArgument,
    IoError,
    InvalidModel,
    UnsupportedModel,
    InternalError
};

struct Error
{
    ErrorCode code = ErrorCode::InternalError;
    std::string message;
};

template<typename T>
class Result
{
public:
    Result(T value) : storage_(std::move(value)) {}
    Result(Error error) : storage_(std::move(error)) {}
    explicit operator bool() const noexcept { return std::holds_alternative<T>(storage_); }
    T& value() & { return std::get<T>(storage_); }
    const T& value() const& { return std::get<T>(storage_); }
    T&& value() && { return std::move(std::get<T>(storage_)); }
    const Error& error() const { return std::get<Error>(storage_); }

private:
    std::variant<T, Error> storage_;
};

template<>
class Result<void>
{
public:
    Result() = default;
    Result(Error error) : failed_(true), error_(std::move(error)) {}
    explicit operator bool() const noexcept { return !failed_; }
    const Error& error() const { return error_; }

private:
    bool failed_ = false;
    Error error_;
};

struct SamplingOptions
{
    float temperature = 1.0f;
    uint32_t top_k = 0;
    float top_p = 1.0f;
    float min_p = 0.0f;
};

struct SampledToken
{
    int32_t token_id = -1;
    float probability = 0.0f;
    bool is_stop_token = false; // StreamToken::is_stop_token of the generate loop (session.h:63-72)
};

enum class RouterScoreFunction
{
    Softmax,
    Sigmoid,
    SqrtSoftplus
};

enum class RouterNormalization
{
    None,
    SelectedExperts
};

struct ExpertRoute
{
    uint32_t token_index = 0;
    uint32_t rank = 0;
    float weight = 0.0f;
};

struct ExpertBatch
{
    uint32_t expert_id = 0;
    std::vector<ExpertRoute> routes;
};

inline constexpr uint32_t ExpertDispatchNormalizeTopKWeights = 1u;

struct ExpertDispatchOptions
{
    uint32_t expert_count = 0;
    uint32_t top_k = 0;
    RouterScoreFunction score_function = RouterScoreFunction::Softmax;
    RouterNormalization normalization = RouterNormalization::SelectedExperts;
    float routed_scaling_factor = 1.0f;
    std::span<const float> selection_bias;
    std::span<const uint32_t> explicit_expert_ids;
    uint32_t flags = ExpertDispatchNormalizeTopKWeights;
};

struct ExpertDispatchPlan
{
    std::vector<ExpertBatch> batches;
    size_t assignment_count = 0;
};

namespace detail {

inline ErrorCode to_error_code(int status_plus_one)
{
    switch (status_plus_one)
    {
    case MOE_STATUS_INVALID_ARGUMENT: return ErrorCode::InvalidArgument;
    case MOE_STATUS_IO_ERROR: return ErrorCode::IoError;
    case MOE_STATUS_INVALID_MODEL: return ErrorCode::InvalidModel;
    case MOE_STATUS_UNSUPPORTED_MODEL: return ErrorCode::UnsupportedModel;
    default: return ErrorCode::InternalError;
    }
}

struct HandleDeleter
{
    void operator()(moe_sampler* handle) const noexcept { moe_sampler_destroy(handle); }
};

using Handle = std::unique_ptr<moe_sampler, HandleDeleter>;

inline Result<Handle> make_handle(int device, uint32_t max_rows, uint32_t max_vocab)
{
    moe_sampler* raw = nullptr;
    const int status = moe_sampler_create(device, max_rows, max_vocab, &raw);
    if (status != MOE_STATUS_OK)
        return Error{ErrorCode::InternalError, "no usable sm_100 CUDA device for the sampler (there is no CPU path)"};
    return Handle(raw);
}

} // namespace detail

// What a decode step hands back to the host, after LogitsOutputMode of the
// reference (include/ncnn/moe/types.h:304-309).  The reference accepts only
// FullLogits today (src/engine/runtime.cpp:579-580); SampledToken is the mode a
// device-side sampler makes possible: the [sessions x vocab] logits stay on the
// GPU that produced them and only {token, probability} per Session returns.
enum class LogitsOutputMode : uint32_t
{
    FullLogits = 0,  // host logits in, DeviceSampler::sample / sample_batch(std::span<const float>, ...)
    SampledToken = 2 // device logits in, DeviceSampler::sample_batch(DeviceLogits, ...)
};

// A [rows x row_stride] logit matrix that lives on the device, e.g. the staged
// LM-head output of src/engine/cpu_executor.cpp:2978-2995 kept on the GPU.
struct DeviceLogits
{
    const void* data = nullptr; // device pointer
    int dtype = MOE_DTYPE_F32;  // MOE_DTYPE_F32 or MOE_DTYPE_BF16
    uint32_t rows = 0;
    uint32_t vocab = 0;
    size_t row_stride = 0;      // elements between rows, >= vocab
    void* stream = nullptr;     // cudaStream_t the producer wrote the logits on
};

// One sampling stream: what a Session is to the reference sampler.  `seed`
// plays the role of SessionOptions::sampling_seed (session.h:283); `session_id`
// distinguishes the streams of one batch; every sample() call advances `step`.
class DeviceSampler
{
public:
    static Result<std::unique_ptr<DeviceSampler>> create(uint64_t seed = 0, uint64_t session_id = 0, uint32_t max_vocab = 1u << 20,
                                                          uint32_t max_rows = 256, int device = 0)
    {
        auto handle = detail::make_handle(device, max_rows, max_vocab);
        if (!handle)
            return handle.error();
        return std::unique_ptr<DeviceSampler>(new DeviceSampler(std::move(handle).value(), seed, session_id, max_rows));
    }

    // Session::sample: one row of host logits, this stream's options.
    [[nodiscard]] Result<SampledToken> sample(std::span<const float> logits, const SamplingOptions& options = {},
                                              std::span<const int32_t> stop_tokens = {})
    {
        if (logits.empty())
            return Error{ErrorCode::InvalidArgument, "cannot sample empty logits"};
        moe_row_params row{options.temperature, options.top_k, options.top_p, options.min_p, seed_, session_id_, step_};
        const int32_t offsets[2] = {0, static_cast<int32_t>(stop_tokens.size())};
        int32_t token = -1;
        float probability = 0.0f;
        uint32_t flags = 0;
        int32_t row_status = 0;
        const int status = moe_sample_batch_host(handle_.get(), logits.data(), MOE_DTYPE_F32, 1, static_cast<uint32_t>(logits.size()), logits.size(), &row,
                                                 stop_tokens.empty() ? nullptr : offsets, stop_tokens.empty() ? nullptr : stop_tokens.data(), &token,
                                                 &probability, &flags, &row_status, nullptr, 0);
        if (status != MOE_STATUS_OK)
            return Error{detail::to_error_code(status), moe_sampler_last_error(handle_.get())};
        if (row_status != MOE_ROW_OK)
            return Error{detail::to_error_code(moe_row_status_error_code(row_status)), moe_row_status_message(row_status)};
        if ((flags & MOE_ROW_FLAG_USED_UNIFORM) != 0)
            ++step_; // like the Session's generator, the stream advances only when a uniform was consumed
        return SampledToken{token, probability, (flags & MOE_ROW_FLAG_STOP_TOKEN) != 0};
    }

    // The cross-Session step: row r of `logits` ([rows x vocab], host) is sampled
    // with options[r]; row ids are session_id + r, so each row has its own stream.
    [[nodiscard]] std::vector<Result<SampledToken>> sample_batch(std::span<const float> logits, uint32_t vocab, std::span<const SamplingOptions> options,
                                                                 std::span<const int32_t> stop_tokens = {})
    {
        const uint32_t rows = static_cast<uint32_t>(options.size());
        std::vector<Result<SampledToken>> results;
        results.reserve(rows);
        if (vocab == 0 || logits.size() != static_cast<size_t>(rows) * vocab || rows > max_rows_)
        {
            const char* text = vocab == 0 ? "cannot sample empty logits" : "logits do not match rows x vocab or exceed the sampler's row capacity";
            for (uint32_t r = 0; r < rows; ++r)
                results.emplace_back(Error{ErrorCode::InvalidArgument, text});
            return results;
        }
        std::vector<moe_row_params> params(rows);
        std::vector<int32_t> offsets(rows + 1);
        std::vector<int32_t> stops;
        for (uint32_t r = 0; r < rows; ++r)
        {
            params[r] = moe_row_params{options[r].temperature, options[r].top_k, options[r].top_p, options[r].min_p, seed_, session_id_ + r, step_};
            offsets[r] = static_cast<int32_t>(stops.size());
            stops.insert(stops.end(), stop_tokens.begin(), stop_tokens.end());
        }
        offsets[rows] = static_cast<int32_t>(stops.size());
        std::vector<int32_t> token(rows), row_status(rows);
        std::vector<float> probability(rows);
        std::vector<uint32_t> flags(rows);
        const int status = moe_sample_batch_host(handle_.get(), logits.data(), MOE_DTYPE_F32, rows, vocab, vocab, params.data(),
                                                 stops.empty() ? nullptr : offsets.data(), stops.empty() ? nullptr : stops.data(), token.data(),
                                                 probability.data(), flags.data(), row_status.data(), nullptr, 0);
        ++step_;
        for (uint32_t r = 0; r < rows; ++r)
        {
            if (status != MOE_STATUS_OK)
                results.emplace_back(Error{detail::to_error_code(status), moe_sampler_last_error(handle_.get())});
            else if (row_status[r] != MOE_ROW_OK)
                results.emplace_back(Error{detail::to_error_code(moe_row_status_error_code(row_status[r])), moe_row_status_message(row_status[r])});
            else
                results.emplace_back(SampledToken{token[r], probability[r], (flags[r] & MOE_ROW_FLAG_STOP_TOKEN) != 0});
        }
        return results;
    }

    // LogitsOutputMode::SampledToken: the cross-Session step on logits that never
    // leave the device.  The sampling kernel is ordered behind the producer on
    // logits.stream; one 16-byte record per row comes back.
    [[nodiscard]] std::vector<Result<SampledToken>> sample_batch(const DeviceLogits& logits, std::span<const SamplingOptions> options,
                                                                 std::span<const int32_t> stop_tokens = {})
    {
        const uint32_t rows = static_cast<uint32_t>(options.size());
        std::vector<Result<SampledToken>> results;
        results.reserve(rows);
        if (logits.data == nullptr || logits.vocab == 0 || logits.rows != rows || rows > max_rows_)
        {
            const char* text = (logits.data == nullptr || logits.vocab == 0) ? "cannot sample empty logits"
                                                                             : "logits do not match the number of options or exceed the sampler's row capacity";
            for (uint32_t r = 0; r < rows; ++r)
                results.emplace_back(Error{ErrorCode::InvalidArgument, text});
            return results;
        }
        std::vector<moe_row_params> params(rows);
        std::vector<int32_t> offsets(rows + 1);
        std::vector<int32_t> stops;
        for (uint32_t r = 0; r < rows; ++r)
        {
            params[r] = moe_row_params{options[r].temperature, options[r].top_k, options[r].top_p, options[r].min_p, seed_, session_id_ + r, step_};
            offsets[r] = static_cast<int32_t>(stops.size());
            stops.insert(stops.end(), stop_tokens.begin(), stop_tokens.end());
        }
        offsets[rows] = static_cast<int32_t>(stops.size());
        if (sampled_rows_ == nullptr)
        {
            void* pinned = nullptr;
            if (moe_host_alloc(sizeof(moe_sampled_row) * max_rows_, &pinned) != MOE_STATUS_OK)
            {
                for (uint32_t r = 0; r < rows; ++r)
                    results.emplace_back(Error{ErrorCode::InternalError, "page-locked result buffer could not be allocated"});
                return results;
            }
            sampled_rows_ = static_cast<moe_sampled_row*>(pinned);
        }
        const int status = moe_sample_tokens(handle_.get(), logits.stream, logits.data, logits.dtype, rows, logits.vocab, logits.row_stride, params.data(), 0,
                                             stops.empty() ? nullptr : offsets.data(), stops.empty() ? nullptr : stops.data(), sampled_rows_);
        ++step_;
        for (uint32_t r = 0; r < rows; ++r)
        {
            const moe_sampled_row& row = sampled_rows_[r];
            if (status != MOE_STATUS_OK)
                results.emplace_back(Error{detail::to_error_code(status), moe_sampler_last_error(handle_.get())});
            else if (row.row_status != MOE_ROW_OK)
                results.emplace_back(Error{detail::to_error_code(moe_row_status_error_code(row.row_status)), moe_row_status_message(row.row_status)});
            else
                results.emplace_back(SampledToken{row.token_id, row.probability, (row.row_flags & MOE_ROW_FLAG_STOP_TOKEN) != 0});
        }
        return results;
    }

    ~DeviceSampler()
    {
        if (sampled_rows_ != nullptr)
            moe_host_free(sampled_rows_);
    }
    DeviceSampler(const DeviceSampler&) = delete;
    DeviceSampler& operator=(const DeviceSampler&) = delete;

    // The verification step of Session::generate's speculative branch
    // (src/engine/session.cpp:776-880): `proposed` tokens of the draft model
    // against target_logits [(proposed.size() + 1) x vocab] and draft_logits
    // [proposed.size() x vocab] (host).  Returns the tokens the reference would
    // emit: the accepted proposals with their reported probabilities, then the
    // token that follows them.  The stream advances by the uniforms consumed.
    [[nodiscard]] Result<std::vector<SampledToken>> verify_speculative(std::span<const float> target_logits, std::span<const float> draft_logits,
                                                                        uint32_t vocab, std::span<const int32_t> proposed, const SamplingOptions& options = {})
    {
        const uint32_t draft_count = static_cast<uint32_t>(proposed.size());
        if (vocab == 0)
            return Error{ErrorCode::InvalidArgument, "cannot sample empty logits"};
        if (draft_count > MOE_SPECULATIVE_MAX_DRAFT || target_logits.size() != static_cast<size_t>(draft_count + 1) * vocab ||
            draft_logits.size() != static_cast<size_t>(draft_count) * vocab)
            return Error{ErrorCode::InvalidArgument, "logits do not match the number of proposed tokens"};
        const moe_row_params row{options.temperature, options.top_k, options.top_p, options.min_p, seed_, session_id_, step_};
        std::vector<float> accepted_probability(draft_count + 1u);
        moe_speculative_result outcome{};
        const int status = moe_speculative_verify_host(handle_.get(), target_logits.data(), draft_count > 0 ? draft_logits.data() : nullptr, MOE_DTYPE_F32,
                                                       draft_count, vocab, vocab, draft_count > 0 ? proposed.data() : nullptr, &row,
                                                       accepted_probability.data(), &outcome);
        if (status != MOE_STATUS_OK)
            return Error{detail::to_error_code(status), moe_sampler_last_error(handle_.get())};
        if (outcome.status != MOE_ROW_OK)
            return Error{detail::to_error_code(moe_row_status_error_code(outcome.status)), moe_row_status_message(outcome.status)};
        step_ += outcome.uniforms_used;
        std::vector<SampledToken> tokens;
        tokens.reserve(outcome.accepted + 1u);
        for (uint32_t index = 0; index < outcome.accepted; ++index)
            tokens.push_back(SampledToken{proposed[index], accepted_probability[index], false});
        tokens.push_back(SampledToken{outcome.next_token, outcome.next_probability, false});
        return tokens;
    }

    [[nodiscard]] uint64_t step() const noexcept { return step_; }
    [[nodiscard]] moe_sampler* native_handle() const noexcept { return handle_.get(); }

private:
    DeviceSampler(detail::Handle handle, uint64_t seed, uint64_t session_id, uint32_t max_rows)
        : handle_(std::move(handle)), seed_(seed), session_id_(session_id), max_rows_(max_rows)
    {
    }

    detail::Handle handle_;
    uint64_t seed_ = 0;
    uint64_t session_id_ = 0;
    uint64_t step_ = 0;
    uint32_t max_rows_ = 0;
    moe_sampled_row* sampled_rows_ = nullptr; // page-locked, max_rows_ records, allocated by the first SampledToken call
};

// ExpertDispatcher on the GPU.  Input is token-major; output is ordered by
// expert id, inside an expert by token then rank, exactly as the reference
// appends routes (src/graph/expert_dispatcher.cpp:110-157).
class DeviceExpertDispatcher
{
public:
    static Result<std::unique_ptr<DeviceExpertDispatcher>> create(int device = 0)
    {
        auto handle = detail::make_handle(device, 1, 1);
        if (!handle)
            return handle.error();
        return std::unique_ptr<DeviceExpertDispatcher>(new DeviceExpertDispatcher(std::move(handle).value()));
    }

    [[nodiscard]] Result<ExpertDispatchPlan> dispatch(std::span<const float> router_logits, uint32_t token_count, const ExpertDispatchOptions& options) const
    {
        ExpertDispatchPlan plan;
        auto status = dispatch_into(router_logits, token_count, options, plan);
        if (!status)
            return status.error();
        return plan;
    }

    // Reuses the caller's plan storage across decode steps.
    [[nodiscard]] Result<void> dispatch_into(std::span<const float> router_logits, uint32_t token_count, const ExpertDispatchOptions& options,
                                             ExpertDispatchPlan& result) const
    {
        moe_router_options native{};
        native.expert_count = options.expert_count;
        native.top_k = options.top_k;
        native.score_function = static_cast<int32_t>(options.score_function);
        native.normalization = static_cast<int32_t>(options.normalization);
        native.routed_scaling_factor = options.routed_scaling_factor;
        native.flags = options.flags;
        native.selection_bias = options.selection_bias.empty() ? nullptr : options.selection_bias.data();
        native.explicit_expert_ids = options.explicit_expert_ids.empty() ? nullptr : options.explicit_expert_ids.data();
        // the size checks of expert_dispatcher.cpp:81-96 that need the spans
        int precheck = moe_router_check_options(token_count, &native);
        if (precheck == 0 || precheck == 109 || precheck == 110)
        {
            if (token_count != 0 && options.expert_count != 0 &&
                (router_logits.size() / options.expert_count != token_count || router_logits.size() % options.expert_count != 0))
                precheck = 106;
            else if (!options.selection_bias.empty() && options.selection_bias.size() != options.expert_count)
                precheck = 107;
            else if (!options.explicit_expert_ids.empty() && options.explicit_expert_ids.size() != static_cast<size_t>(token_count) * options.top_k)
                precheck = 108;
        }
        if (precheck != 0)
            return Error{detail::to_error_code(moe_router_status_error_code(precheck)), moe_router_status_message(precheck)};

        const size_t routes = static_cast<size_t>(token_count) * options.top_k;
        offsets_.resize(static_cast<size_t>(options.expert_count) + 1);
        token_.resize(routes);
        rank_.resize(routes);
        weight_.resize(routes);
        int32_t plan_status = 0;
        const int status = moe_router_dispatch_host(handle_.get(), router_logits.data(), token_count, &native, offsets_.data(), token_.data(), rank_.data(),
                                                    weight_.data(), &plan_status);
        if (plan_status != 0)
            return Error{detail::to_error_code(moe_router_status_error_code(plan_status)), moe_router_status_message(plan_status)};
        if (status != MOE_STATUS_OK)
            return Error{detail::to_error_code(status), moe_sampler_last_error(handle_.get())};

        size_t used = 0;
        for (uint32_t expert = 0; expert < options.expert_count; ++expert)
        {
            const uint32_t begin = offsets_[expert];
            const uint32_t end = offsets_[expert + 1];
            if (begin == end)
                continue;
            if (result.batches.size() <= used)
                result.batches.emplace_back();
            ExpertBatch& batch = result.batches[used++];
            batch.expert_id = expert;
            batch.routes.resize(end - begin);
            for (uint32_t i = begin; i < end; ++i)
                batch.routes[i - begin] = ExpertRoute{token_[i], rank_[i], weight_[i]};
        }
        result.batches.resize(used);
        result.assignment_count = routes;
        return {};
    }

private:
    explicit DeviceExpertDispatcher(detail::Handle handle) : handle_(std::move(handle)) {}

    detail::Handle handle_;
    mutable std::vector<uint32_t> offsets_, token_, rank_;
    mutable std::vector<float> weight_;
};

} // namespace moe_b200
