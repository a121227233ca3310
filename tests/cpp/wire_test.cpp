// The JSONL wire path (ncnn-moe-runtime_b200/host/moe_b200_wire.hpp): request
// lines in the reference worker's format, one batched sampling call per decode
// step for all generations in flight, token / done events out.  Expected tokens
// come from DeviceSampler::sample on the same rows with the same seeds.
#include <cstdio>
#include <source_location>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../ncnn-moe-runtime_b200/host/moe_b200_wire.hpp"

using namespace moe_b200;

extern "C" {
int cudaMalloc(void** pointer, size_t bytes);
int cudaFree(void* pointer);
int cudaMemcpy(void* destination, const void* source, size_t bytes, int kind);
}

static void check(bool condition, const std::source_location where = std::source_location::current())
{
    if (!condition)
        throw std::runtime_error(std::string("check failed at line ") + std::to_string(where.line()));
}

static bool contains(const std::string& text, const std::string& part)
{
    return text.find(part) != std::string::npos;
}

static std::vector<float> make_logits(uint32_t rows, uint32_t vocab, uint32_t seed)
{
    std::vector<float> logits(static_cast<size_t>(rows) * vocab);
    uint32_t state = seed;
    for (float& value : logits)
    {
        state = state * 1664525u + 1013904223u;
        value = static_cast<float>(state >> 8) * (10.0f / 16777216.0f) - 5.0f;
    }
    return logits;
}

int main()
{
    try
    {
        constexpr uint32_t vocab = 7001;
        auto created = WireSamplingRouter::create(vocab, 8);
        check(static_cast<bool>(created));
        WireSamplingRouter& router = *created.value();

        // field parsing, defaults and the reference's messages
        check(contains(router.handle_line(R"({"op":"create_session","session_id":"a","seed":11})")[0], "\"event\":\"session_created\""));
        check(contains(router.handle_line(R"({"op":"create_session","session_id":"b","seed":12,"prefill_chunk_size":256})")[0], "session_created"));
        check(contains(router.handle_line(R"({"op":"create_session","session_id":"c"})")[0], "session_created"));
        check(contains(router.handle_line(R"({"op":"create_session","session_id":"a"})")[0], "session already exists"));
        check(contains(router.handle_line(R"({"op":"generate","session_id":"nobody"})")[0], "unknown session: nobody"));
        check(contains(router.handle_line(R"({"op":"generate","session_id":"a","top_p":0.0})")[0], "top_p must be in the range (0, 1]"));
        check(contains(router.handle_line(R"({"op":"generate","session_id":"a","temperature":-1})")[0], "temperature must be finite and non-negative"));
        check(router.active().empty());

        // three generations in flight at once, each with its own parameters
        check(router.handle_line(R"({"op":"generate","request_id":"r-a","session_id":"a","prompt_tokens":[1,2,3],"max_new_tokens":3,"temperature":0.8,"top_k":40,"top_p":0.95,"min_p":0.0,"stop_tokens":[]})").empty());
        check(router.handle_line(R"({"op":"generate","request_id":"r-b","session_id":"b","max_new_tokens":2})").empty()); // no temperature: greedy
        check(router.handle_line(R"({"op":"generate","request_id":"r-c","session_id":"c","max_new_tokens":5,"temperature":1.0,"top_k":5,"stop_tokens":[4242, 17]})").empty());
        check(contains(router.handle_line(R"({"op":"generate","request_id":"again","session_id":"a"})")[0], "already has a generation in flight"));
        check(router.active().size() == 3);
        check(router.active()[1].sampling.temperature == 0.0f && router.active()[1].sampling.top_p == 1.0f);
        check(router.active()[2].stop_tokens.size() == 2 && router.active()[2].stop_tokens[1] == 17);

        // the same rows through Session-shaped samplers: seed of the session, row id = position in the session table
        auto session_a = DeviceSampler::create(11, 0, vocab, 1);
        auto session_b = DeviceSampler::create(12, 1, vocab, 1);
        auto session_c = DeviceSampler::create(0, 2, vocab, 1);
        SamplingOptions options_a{0.8f, 40, 0.95f, 0.0f};
        SamplingOptions options_b{0.0f, 0, 1.0f, 0.0f};
        SamplingOptions options_c{1.0f, 5, 1.0f, 0.0f};

        void* device_logits = nullptr;
        check(cudaMalloc(&device_logits, sizeof(float) * 3 * vocab) == 0);
        uint32_t produced_a = 0, produced_b = 0;
        for (uint32_t step = 0; step < 3; ++step)
        {
            const uint32_t rows = static_cast<uint32_t>(router.active().size());
            std::vector<float> logits = make_logits(rows, vocab, 100 + step);
            if (step == 1)
                logits[(rows - 1) * static_cast<size_t>(vocab) + 4242] = 60.0f; // session c meets one of its stop tokens
            check(cudaMemcpy(device_logits, logits.data(), sizeof(float) * logits.size(), 1) == 0);
            DeviceLogits view{device_logits, MOE_DTYPE_F32, rows, vocab, vocab, nullptr};
            const auto order = router.active(); // copy: step() retires finished requests
            const std::vector<std::string> events = router.step(view);
            size_t cursor = 0;
            for (uint32_t r = 0; r < rows; ++r)
            {
                const std::span<const float> row(logits.data() + static_cast<size_t>(r) * vocab, vocab);
                Result<SampledToken> expected = Error{ErrorCode::InternalError, "unset"};
                if (order[r].session_id == "a")
                    expected = session_a.value()->sample(row, options_a), ++produced_a;
                else if (order[r].session_id == "b")
                    expected = session_b.value()->sample(row, options_b), ++produced_b;
                else
                    expected = session_c.value()->sample(row, options_c, std::vector<int32_t>{4242, 17});
                check(static_cast<bool>(expected));
                const std::string& token_event = events.at(cursor++);
                check(contains(token_event, "\"event\":\"token\"") && contains(token_event, "\"request_id\":\"" + order[r].request_id + "\""));
                check(contains(token_event, "\"token_id\":" + std::to_string(expected.value().token_id) + ","));
                check(contains(token_event, "\"index\":" + std::to_string(order[r].generated) + ","));
                check(contains(token_event, std::string("\"is_stop_token\":") + (expected.value().is_stop_token ? "true" : "false")));
                const bool ends = expected.value().is_stop_token || order[r].generated + 1 >= order[r].max_new_tokens;
                if (ends)
                {
                    const std::string& done = events.at(cursor++);
                    check(contains(done, "\"event\":\"done\"") && contains(done, "\"request_id\":\"" + order[r].request_id + "\""));
                    check(contains(done, std::string("\"stopped_by_stop_token\":") + (expected.value().is_stop_token ? "true" : "false")));
                    check(contains(done, "\"generated_tokens\":" + std::to_string(order[r].generated + 1)));
                }
            }
            check(cursor == events.size());
        }
        check(produced_a == 3 && produced_b == 2);
        check(router.active().empty()); // a: 3 tokens, b: 2 tokens, c: stopped by token 4242 at its second step

        // cancel
        check(router.handle_line(R"({"op":"generate","request_id":"long","session_id":"b","max_new_tokens":1000,"temperature":0.5})").empty());
        const auto cancelled = router.handle_line(R"({"op":"cancel","request_id":"long"})");
        check(cancelled.size() == 2 && contains(cancelled[0], "cancel_requested") && contains(cancelled[1], "\"cancelled\":true"));
        check(router.active().empty());
        check(contains(router.handle_line(R"({"op":"cancel","request_id":"long"})")[0], "no generation is active"));
        check(cudaFree(device_logits) == 0);
    }
    catch (const std::exception& error)
    {
        std::fprintf(stderr, "%s\n", error.what());
        return 1;
    }
    std::puts("all wire tests passed");
    return 0;
}
