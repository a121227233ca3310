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
    }
    catch (const std::exception& error)
    {
        std::fprintf(stderr, "%s\n", error.what());
        return 1;
    }
    std::puts("all adapter tests passed");
    return 0;
}
