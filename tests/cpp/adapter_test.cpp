// Exercises the C++20 adapter the way the reference's own tests exercise
// Session::sample and ExpertDispatcher (tests/test_runtime.cpp:4320-4362 and
// :3366-3539 of the reference): same inputs, same expectations, GPU underneath.
#include <array>
#include <cmath>
#include <cstdio>
#include <limits>
#include <source_location>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../ncnn-moe-runtime_b200/host/moe_b200.hpp"

using namespace moe_b200;

// The CUDA runtime calls this test needs to put logits on the device (the
// adapter itself needs no CUDA header): declared here, resolved from libcudart.
extern "C" {
int cudaMalloc(void** pointer, size_t bytes);
int cudaFree(void* pointer);
int cudaMemcpy(void* destination, const void* source, size_t bytes, int kind);
}
constexpr int kCudaMemcpyHostToDevice = 1;

static void check(bool condition, const std::source_location where = std::source_location::current())
{
    if (!condition)
        throw std::runtime_error(std::string("check failed at line ") + std::to_string(where.line()));
}

static void check_near(float actual, float expected, float tolerance, const std::source_location where = std::source_location::current())
{
    check(std::fabs(actual - expected) <= tolerance, where);
}

static void test_sampling()
{
    auto created = DeviceSampler::create(1234);
    check(static_cast<bool>(created));
    DeviceSampler& session = *created.value();

    std::vector<float> logits = {1.0f, 2.0f, 3.0f};
    SamplingOptions greedy_options;
    greedy_options.temperature = 0.0f;
    auto greedy = session.sample(logits, greedy_options);
    check(static_cast<bool>(greedy));
    check(greedy.value().token_id == 2);
    check_near(greedy.value().probability, 1.0f, 1e-6f);

    logits = {3.0f, std::numeric_limits<float>::quiet_NaN(), 3.0f};
    greedy = session.sample(logits, greedy_options);
    check(static_cast<bool>(greedy));
    check(greedy.value().token_id == 0);

    logits = {std::numeric_limits<float>::quiet_NaN(), std::numeric_limits<float>::infinity()};
    greedy = session.sample(logits, greedy_options);
    check(!greedy);
    check(greedy.error().code == ErrorCode::InvalidArgument);
    check(greedy.error().message == "sampling requires at least one finite logit");

    logits = {1.0f, 2.0f, 3.0f};
    SamplingOptions top_k_options;
    top_k_options.top_k = 1;
    auto top_k = session.sample(logits, top_k_options);
    check(static_cast<bool>(top_k));
    check(top_k.value().token_id == 2);
    check(session.step() == 0); // a single-candidate distribution consumes no uniform

    SamplingOptions invalid_options;
    invalid_options.top_p = 0.0f;
    auto invalid = session.sample(logits, invalid_options);
    check(!invalid);
    check(invalid.error().code == ErrorCode::InvalidArgument);
    check(invalid.error().message == "top_p must be in the range (0, 1]");

    auto empty = session.sample(std::span<const float>{});
    check(!empty && empty.error().message == "cannot sample empty logits");

    // a real draw advances the stream, and the stop list flags the emitted token
    SamplingOptions hot;
    hot.temperature = 5.0f;
    const std::array<int32_t, 3> stops = {0, 1, 2};
    auto drawn = session.sample(logits, hot, stops);
    check(static_cast<bool>(drawn));
    check(drawn.value().is_stop_token);
    check(session.step() == 1);

    // one cross-Session step with per-row options
    const std::vector<float> batch = {1, 2, 3, 9, 0, 0, 0, 0, 7};
    const std::vector<SamplingOptions> options = {greedy_options, top_k_options, invalid_options};
    auto results = session.sample_batch(batch, 3, options);
    check(results.size() == 3);
    check(results[0] && results[0].value().token_id == 2);
    check(results[1] && results[1].value().token_id == 0);
    check(!results[2] && results[2].error().code == ErrorCode::InvalidArgument);
}

static void test_expert_dispatcher()
{
    auto created = DeviceExpertDispatcher::create();
    check(static_cast<bool>(created));
    DeviceExpertDispatcher& dispatcher = *created.value();

    ExpertDispatchOptions options;
    options.expert_count = 6;
    options.top_k = 1;
    const std::vector<float> logits = {0, 5, 0, 0, 0, 1, 0, 1, 0, 0, 0, 5, 0, 4, 0, 0, 0, 1, 0, 1, 0, 0, 0, 4};
    auto dispatch = dispatcher.dispatch(logits, 4, options);
    check(static_cast<bool>(dispatch));
    check(dispatch.value().assignment_count == 4);
    check(dispatch.value().batches.size() == 2);
    check(dispatch.value().batches[0].expert_id == 1);
    check(dispatch.value().batches[0].routes.size() == 2);
    check(dispatch.value().batches[0].routes[0].token_index == 0);
    check(dispatch.value().batches[0].routes[1].token_index == 2);
    check_near(dispatch.value().batches[0].routes[0].weight, 1.0f, 1e-6f);
    check(dispatch.value().batches[1].expert_id == 5);
    check(dispatch.value().batches[1].routes[0].token_index == 1);
    check(dispatch.value().batches[1].routes[1].token_index == 3);

    options.expert_count = 3;
    options.top_k = 2;
    const std::vector<float> weighted_logits = {2.0f, 1.0f, 0.0f};
    auto weighted = dispatcher.dispatch(weighted_logits, 1, options);
    check(static_cast<bool>(weighted));
    check(weighted.value().batches.size() == 2);
    check(weighted.value().batches[0].routes[0].rank == 0);
    check(weighted.value().batches[1].routes[0].rank == 1);
    check_near(weighted.value().batches[0].routes[0].weight + weighted.value().batches[1].routes[0].weight, 1.0f, 1e-6f);

    ExpertDispatchPlan reusable;
    auto into = dispatcher.dispatch_into(weighted_logits, 1, options, reusable);
    check(static_cast<bool>(into));
    check(reusable.batches.size() == weighted.value().batches.size());
    const ExpertBatch* reused_batches = reusable.batches.data();
    const ExpertRoute* reused_route = reusable.batches.front().routes.data();
    const std::vector<float> next_logits = {0.0f, 1.0f, 2.0f};
    into = dispatcher.dispatch_into(next_logits, 1, options, reusable);
    check(static_cast<bool>(into));
    check(reusable.batches.data() == reused_batches);             // storage is reused across decode steps
    check(reusable.batches.front().routes.data() == reused_route);

    const std::vector<float> invalid_logits = {1.0f, 2.0f};
    auto invalid = dispatcher.dispatch(invalid_logits, 1, options);
    check(!invalid);
    check(invalid.error().code == ErrorCode::InvalidArgument);
    check(invalid.error().message == "router logits shape does not match token and expert counts");

    // sqrt-softplus with a selection bias that picks the expert but stays out of the weight
    ExpertDispatchOptions deepseek;
    deepseek.expert_count = 4;
    deepseek.top_k = 2;
    deepseek.score_function = RouterScoreFunction::SqrtSoftplus;
    deepseek.routed_scaling_factor = 1.5f;
    const std::array<float, 4> selection_bias = {0.0f, 100.0f, 0.0f, 0.0f};
    deepseek.selection_bias = selection_bias;
    const std::array<float, 4> deepseek_logits = {4.0f, -4.0f, 3.0f, 2.0f};
    auto routed = dispatcher.dispatch(deepseek_logits, 1, deepseek);
    check(static_cast<bool>(routed));
    check(routed.value().batches.size() == 2);
    check(routed.value().batches[0].expert_id == 0);
    check(routed.value().batches[1].expert_id == 1);
    check_near(routed.value().batches[0].routes[0].weight + routed.value().batches[1].routes[0].weight, 1.5f, 1e-5f);

    const std::array<uint32_t, 2> explicit_experts = {3, 2};
    deepseek.selection_bias = {};
    deepseek.explicit_expert_ids = explicit_experts;
    routed = dispatcher.dispatch(deepseek_logits, 1, deepseek);
    check(static_cast<bool>(routed));
    check(routed.value().batches[0].expert_id == 2);
    check(routed.value().batches[1].expert_id == 3);
}

// LogitsOutputMode::SampledToken: the same rows sampled from logits that stay on
// the device must give what the host-logits path (FullLogits) gives, stop flags
// and per-row errors included.
static void test_device_resident_logits()
{
    constexpr uint32_t rows = 6, vocab = 5000;
    std::vector<float> logits(static_cast<size_t>(rows) * vocab);
    uint32_t state = 12345u;
    for (float& value : logits)
    {
        state = state * 1664525u + 1013904223u;
        value = static_cast<float>(state >> 8) * (12.0f / 16777216.0f) - 6.0f;
    }
    logits[3 * vocab + 77] = 40.0f; // row 3 collapses to one candidate
    std::vector<SamplingOptions> options(rows);
    options[0].temperature = 0.0f;
    options[1].top_k = 40;
    options[1].top_p = 0.9f;
    options[2].top_k = 5;
    options[2].temperature = 0.7f;
    options[3].top_p = 0.95f;
    options[4].top_p = 0.0f; // invalid: reported per row
    options[5].top_k = 300;
    options[5].min_p = 0.01f;
    const std::array<int32_t, 1> stops = {77};

    auto host_side = DeviceSampler::create(99, 7, vocab, rows);
    auto device_side = DeviceSampler::create(99, 7, vocab, rows);
    check(static_cast<bool>(host_side) && static_cast<bool>(device_side));
    const auto expected = host_side.value()->sample_batch(logits, vocab, options, stops);

    void* device_logits = nullptr;
    check(cudaMalloc(&device_logits, logits.size() * sizeof(float)) == 0);
    check(cudaMemcpy(device_logits, logits.data(), logits.size() * sizeof(float), kCudaMemcpyHostToDevice) == 0);
    DeviceLogits view;
    view.data = device_logits;
    view.dtype = MOE_DTYPE_F32;
    view.rows = rows;
    view.vocab = vocab;
    view.row_stride = vocab;
    view.stream = nullptr; // the legacy default stream: the copy above has completed
    const auto sampled = device_side.value()->sample_batch(view, options, stops);
    check(sampled.size() == rows && expected.size() == rows);
    for (uint32_t r = 0; r < rows; ++r)
    {
        check(static_cast<bool>(sampled[r]) == static_cast<bool>(expected[r]));
        if (!sampled[r])
        {
            check(sampled[r].error().code == expected[r].error().code);
            check(sampled[r].error().message == expected[r].error().message);
            continue;
        }
        check(sampled[r].value().token_id == expected[r].value().token_id);
        check(sampled[r].value().probability == expected[r].value().probability);
        check(sampled[r].value().is_stop_token == expected[r].value().is_stop_token);
    }
    check(!sampled[4] && sampled[4].error().message == "top_p must be in the range (0, 1]");
    check(sampled[3].value().token_id == 77 && sampled[3].value().is_stop_token);
    check(device_side.value()->step() == 1);
    check(cudaFree(device_logits) == 0);
}

// The verification step of speculative decoding (src/engine/session.cpp:776-880
// of the reference) on cases small enough to follow by hand.
static void test_speculative_verification()
{
    auto created = DeviceSampler::create(77, 0, 1u << 12, 64);
    check(static_cast<bool>(created));
    DeviceSampler& session = *created.value();
    const uint32_t vocab = 3;

    // greedy: proposals are accepted while they equal the target's best token (:778-794)
    SamplingOptions greedy;
    greedy.temperature = 0.0f;
    const std::vector<float> target = {0.0f, 5.0f, 1.0f, 9.0f, 0.0f, 0.0f, 0.0f, 0.0f, 7.0f};
    const std::vector<float> draft = {0.0f, 4.0f, 0.0f, 3.0f, 0.0f, 0.0f};
    std::vector<int32_t> proposed = {1, 0};
    auto emitted = session.verify_speculative(target, draft, vocab, proposed, greedy);
    check(static_cast<bool>(emitted));
    check(emitted.value().size() == 3);
    check(emitted.value()[0].token_id == 1 && emitted.value()[1].token_id == 0 && emitted.value()[2].token_id == 2);
    check_near(emitted.value()[0].probability, 1.0f, 0.0f);
    check_near(emitted.value()[2].probability, 1.0f, 0.0f);
    check(session.step() == 0); // greedy consumes no uniform

    proposed = {1, 2};
    emitted = session.verify_speculative(target, draft, vocab, proposed, greedy);
    check(static_cast<bool>(emitted));
    check(emitted.value().size() == 2);
    check(emitted.value()[0].token_id == 1 && emitted.value()[1].token_id == 0); // the target's own token replaces the wrong proposal

    // identical models: the acceptance probability is 1, every proposal passes (:822-835)
    SamplingOptions plain;
    const std::vector<float> flat(9, 0.0f);
    const std::vector<float> flat_draft(6, 0.0f);
    proposed = {2, 0};
    emitted = session.verify_speculative(flat, flat_draft, vocab, proposed, plain);
    check(static_cast<bool>(emitted));
    check(emitted.value().size() == 3);
    check(emitted.value()[0].token_id == 2 && emitted.value()[1].token_id == 0);
    check_near(emitted.value()[0].probability, 1.0f / 3.0f, 1e-6f);
    check_near(emitted.value()[2].probability, 1.0f / 3.0f, 1e-6f);
    check(session.step() == 3); // two acceptance tests and the sample of the third row

    // a proposal the draft distribution does not contain is the reference's internal error (:813-821)
    SamplingOptions top_one;
    top_one.top_k = 1;
    proposed = {2, 0};
    emitted = session.verify_speculative(target, draft, vocab, proposed, top_one);
    check(!emitted);
    check(emitted.error().code == ErrorCode::InternalError);
    check(emitted.error().message == "sampled draft token has zero probability");

    // models that disagree completely: the proposal is rejected (unless the uniform is below 5e-5)
    // and the residual max(0, target - draft) has all its mass on the target's token (:150-202)
    const std::vector<float> sure_target = {10.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    const std::vector<float> sure_draft = {0.0f, 10.0f, 0.0f};
    proposed = {1};
    const uint64_t before = session.step();
    emitted = session.verify_speculative(sure_target, sure_draft, vocab, proposed, plain);
    check(static_cast<bool>(emitted));
    check(emitted.value().size() == 1);
    check(emitted.value()[0].token_id == 0);
    check_near(emitted.value()[0].probability, 1.0f, 1e-6f);
    check(session.step() == before + 2); // the acceptance test and the residual draw

    // shape errors are values too
    emitted = session.verify_speculative(sure_target, sure_draft, vocab, std::vector<int32_t>{1, 1}, plain);
    check(!emitted);
    check(emitted.error().code == ErrorCode::InvalidArgument);
}

int main()
{
    try
    {
        test_sampling();
        test_expert_dispatcher();
        test_speculative_verification();
        test_device_resident_logits();
    }
    catch (const std::exception& error)
    {
        std::fprintf(stderr, "%s\n", error.what());
        return 1;
    }
    std::puts("all adapter tests passed");
    return 0;
}
