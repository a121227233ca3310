// JSONL wire path for the batched sampler: the request fields of the reference's
// worker protocol (examples/ncnn_moe_worker.cpp:1030-1069, client side
// tools/ncnn_moe_protocol.py:140-177) routed into ONE sampling call per decode
// step for all generations that are in flight.
//
// The reference worker parses a `generate` request into GenerationOptions and
// then runs that one generation to completion on a thread of its own; a second
// `generate` is refused until the first has finished (:1033-1034).  With the
// sampler on the GPU the step that matters is shared: every active generation
// contributes one row of the [sessions x vocab] logit matrix, and all rows are
// sampled with their own parameters in one launch (moe_sample_tokens).  This
// header is that piece and nothing else: it keeps the table of sessions and
// active requests, turns request lines into per-row parameters with the
// worker's field names and defaults, and turns the sampled rows back into the
// worker's `token` / `done` events.  Prefill and the forward pass stay with the
// engine that owns the model; it calls step() with the logits it produced.
//
// Accepted lines (one JSON object each, flat, as the reference client writes them):
//   {"op":"create_session","session_id":"a","seed":7}
//   {"op":"generate","request_id":"r1","session_id":"a","max_new_tokens":64,
//    "temperature":0.8,"top_k":40,"top_p":0.95,"min_p":0.0,"stop_tokens":[2]}
//   {"op":"cancel","request_id":"r1"}
// Field defaults are the worker's: request_id "generate", session_id "main",
// temperature 0 when absent (greedy), top_k 0, top_p 1, min_p 0, no stop tokens,
// max_new_tokens of GenerationOptions (include/ncnn/moe/session.h:74-86).
#pragma once

#include <algorithm>
#include <charconv>
#include <cstdio>
#include <cstdlib>
#include <optional>
#include <string>
#include <string_view>
#include <vector>

#include "moe_b200.hpp"

namespace moe_b200 {

namespace wire_detail {

// Value text of `key` in a flat JSON object, or nothing.  Strings come back
// without their quotes (escapes other than \" and \\ are not used by the protocol's ids).
inline std::optional<std::string_view> raw_value(std::string_view object, std::string_view key)
{
    const std::string quoted = "\"" + std::string(key) + "\"";
    size_t at = 0;
    while ((at = object.find(quoted, at)) != std::string_view::npos)
    {
        size_t cursor = at + quoted.size();
        while (cursor < object.size() && (object[cursor] == ' ' || object[cursor] == '\t'))
            ++cursor;
        if (cursor >= object.size() || object[cursor] != ':')
        {
            at += quoted.size();
            continue; // the text was a value, not a key
        }
        ++cursor;
        while (cursor < object.size() && (object[cursor] == ' ' || object[cursor] == '\t'))
            ++cursor;
        if (cursor >= object.size())
            return std::nullopt;
        if (object[cursor] == '"')
        {
            size_t end = cursor + 1;
            while (end < object.size() && object[end] != '"')
                end += (object[end] == '\\') ? 2 : 1;
            return object.substr(cursor + 1, std::min(end, object.size()) - cursor - 1);
        }
        if (object[cursor] == '[')
        {
            const size_t end = object.find(']', cursor);
            return object.substr(cursor, (end == std::string_view::npos ? object.size() : end + 1) - cursor);
        }
        size_t end = cursor;
        while (end < object.size() && object[end] != ',' && object[end] != '}' && object[end] != ' ')
            ++end;
        return object.substr(cursor, end - cursor);
    }
    return std::nullopt;
}

inline std::optional<double> number(std::string_view object, std::string_view key)
{
    const auto text = raw_value(object, key);
    if (!text || text->empty())
        return std::nullopt;
    const std::string copy(*text);
    char* end = nullptr;
    const double value = std::strtod(copy.c_str(), &end);
    if (end == copy.c_str())
        return std::nullopt;
    return value;
}

inline std::vector<int32_t> token_list(std::string_view object, std::string_view key)
{
    std::vector<int32_t> tokens;
    const auto text = raw_value(object, key);
    if (!text || text->size() < 2 || text->front() != '[')
        return tokens;
    const char* cursor = text->data() + 1;
    const char* const end = text->data() + text->size();
    while (cursor < end)
    {
        while (cursor < end && (*cursor == ' ' || *cursor == ','))
            ++cursor;
        int32_t value = 0;
        const auto parsed = std::from_chars(cursor, end, value);
        if (parsed.ec != std::errc())
            break;
        tokens.push_back(value);
        cursor = parsed.ptr;
    }
    return tokens;
}

inline std::string escape(std::string_view text)
{
    std::string out;
    for (const char c : text)
    {
        if (c == '"' || c == '\\')
            out.push_back('\\');
        out.push_back(c);
    }
    return out;
}

inline std::string error_event(std::string_view request_id, std::string_view message)
{
    return "{\"event\":\"error\",\"request_id\":\"" + escape(request_id) + "\",\"message\":\"" + escape(message) + "\"}";
}

} // namespace wire_detail

class WireSamplingRouter
{
public:
    struct ActiveRequest
    {
        std::string request_id;
        std::string session_id;
        size_t session = 0; // position in the session table = the row id of the session's random stream
        SamplingOptions sampling;
        std::vector<int32_t> stop_tokens;
        uint32_t max_new_tokens = 0;
        uint32_t generated = 0;
        bool cancelled = false;
    };

    static Result<std::unique_ptr<WireSamplingRouter>> create(uint32_t max_vocab, uint32_t max_sessions = 256, int device = 0)
    {
        auto handle = detail::make_handle(device, max_sessions, max_vocab);
        if (!handle)
            return handle.error();
        return std::unique_ptr<WireSamplingRouter>(new WireSamplingRouter(std::move(handle).value(), max_sessions));
    }

    ~WireSamplingRouter()
    {
        if (sampled_rows_ != nullptr)
            moe_host_free(sampled_rows_);
    }
    WireSamplingRouter(const WireSamplingRouter&) = delete;
    WireSamplingRouter& operator=(const WireSamplingRouter&) = delete;

    // One request line in, the event lines it produces at once out (token events come from step()).
    std::vector<std::string> handle_line(std::string_view line)
    {
        using namespace wire_detail;
        std::vector<std::string> events;
        const std::string op(raw_value(line, "op").value_or(""));
        if (op == "create_session")
        {
            const auto session_id = raw_value(line, "session_id");
            if (!session_id)
                return {error_event("", "create_session requires session_id")};
            if (find_session(*session_id) != sessions_.size())
                return {error_event("", "session already exists: " + std::string(*session_id))};
            if (sessions_.size() >= max_sessions_)
                return {error_event("", "session table is full")};
            sessions_.push_back(SessionEntry{std::string(*session_id), static_cast<uint64_t>(number(line, "seed").value_or(0.0)), 0});
            events.push_back("{\"event\":\"session_created\",\"session_id\":\"" + escape(*session_id) + "\"}");
        }
        else if (op == "generate")
        {
            ActiveRequest request;
            request.request_id = std::string(raw_value(line, "request_id").value_or("generate"));
            request.session_id = std::string(raw_value(line, "session_id").value_or("main"));
            request.session = find_session(request.session_id);
            if (request.session == sessions_.size())
                return {error_event(request.request_id, "unknown session: " + request.session_id)};
            for (const ActiveRequest& other : active_)
                if (other.session == request.session)
                    return {error_event(request.request_id, "session already has a generation in flight; cancel it first")};
            // the worker's defaults: greedy unless a temperature is given, the other fields as in SamplingOptions
            request.sampling.temperature = static_cast<float>(number(line, "temperature").value_or(0.0));
            request.sampling.top_k = static_cast<uint32_t>(std::max(0.0, number(line, "top_k").value_or(0.0)));
            request.sampling.top_p = static_cast<float>(number(line, "top_p").value_or(1.0));
            request.sampling.min_p = static_cast<float>(number(line, "min_p").value_or(0.0));
            request.stop_tokens = token_list(line, "stop_tokens");
            request.max_new_tokens = static_cast<uint32_t>(std::max(0.0, number(line, "max_new_tokens").value_or(1024.0)));
            // options are refused up front, with the reference's messages (session.cpp:65-74,461-473)
            const moe_row_params probe{request.sampling.temperature, request.sampling.top_k, request.sampling.top_p, request.sampling.min_p, 0, 0, 0};
            const int invalid = validate(probe);
            if (invalid != MOE_ROW_OK)
                return {error_event(request.request_id, moe_row_status_message(invalid))};
            if (request.max_new_tokens == 0)
                events.push_back(done_event(request, false));
            else
                active_.push_back(std::move(request));
        }
        else if (op == "cancel")
        {
            const std::string request_id(raw_value(line, "request_id").value_or(""));
            bool found = false;
            for (ActiveRequest& request : active_)
                if (request_id.empty() || request.request_id == request_id)
                {
                    request.cancelled = true;
                    found = true;
                }
            if (!found)
                return {error_event(request_id, active_.empty() ? "no generation is active" : "request_id does not match an active generation")};
            events.push_back("{\"event\":\"cancel_requested\",\"request_id\":\"" + escape(request_id) + "\"}");
            retire_cancelled(events);
        }
        else
        {
            events.push_back(error_event("", "unknown op: " + op));
        }
        return events;
    }

    // The generations in flight, in the row order step() expects its logits in.
    [[nodiscard]] const std::vector<ActiveRequest>& active() const noexcept { return active_; }

    // One decode step for every active generation: row r of `logits` belongs to active()[r].
    std::vector<std::string> step(const DeviceLogits& logits)
    {
        std::vector<std::string> events;
        const uint32_t rows = static_cast<uint32_t>(active_.size());
        if (rows == 0)
            return events;
        if (logits.data == nullptr || logits.rows != rows || logits.vocab == 0)
        {
            for (const ActiveRequest& request : active_)
                events.push_back(wire_detail::error_event(request.request_id, "logits do not match the generations in flight"));
            return events;
        }
        params_.resize(rows);
        stop_offsets_.resize(rows + 1);
        stop_tokens_.clear();
        for (uint32_t r = 0; r < rows; ++r)
        {
            const ActiveRequest& request = active_[r];
            const SessionEntry& session = sessions_[request.session];
            params_[r] = moe_row_params{request.sampling.temperature, request.sampling.top_k, request.sampling.top_p, request.sampling.min_p,
                                        session.seed, static_cast<uint64_t>(request.session), session.uniforms_drawn};
            stop_offsets_[r] = static_cast<int32_t>(stop_tokens_.size());
            stop_tokens_.insert(stop_tokens_.end(), request.stop_tokens.begin(), request.stop_tokens.end());
        }
        stop_offsets_[rows] = static_cast<int32_t>(stop_tokens_.size());
        if (sampled_rows_ == nullptr)
        {
            void* pinned = nullptr;
            if (moe_host_alloc(sizeof(moe_sampled_row) * max_sessions_, &pinned) != MOE_STATUS_OK)
                return {wire_detail::error_event("", "page-locked result buffer could not be allocated")};
            sampled_rows_ = static_cast<moe_sampled_row*>(pinned);
        }
        const int status = moe_sample_tokens(handle_.get(), logits.stream, logits.data, logits.dtype, rows, logits.vocab, logits.row_stride, params_.data(), 0,
                                             stop_tokens_.empty() ? nullptr : stop_offsets_.data(), stop_tokens_.empty() ? nullptr : stop_tokens_.data(),
                                             sampled_rows_);
        if (status != MOE_STATUS_OK)
        {
            for (const ActiveRequest& request : active_)
                events.push_back(wire_detail::error_event(request.request_id, moe_sampler_last_error(handle_.get())));
            active_.clear();
            return events;
        }
        std::vector<ActiveRequest> still_active;
        still_active.reserve(rows);
        for (uint32_t r = 0; r < rows; ++r)
        {
            ActiveRequest& request = active_[r];
            const moe_sampled_row& row = sampled_rows_[r];
            if (row.row_status != MOE_ROW_OK)
            {
                events.push_back(wire_detail::error_event(request.request_id, moe_row_status_message(row.row_status)));
                continue;
            }
            if ((row.row_flags & MOE_ROW_FLAG_USED_UNIFORM) != 0)
                ++sessions_[request.session].uniforms_drawn; // the session's stream advances only when a uniform was consumed
            const bool is_stop = (row.row_flags & MOE_ROW_FLAG_STOP_TOKEN) != 0;
            char text[96];
            std::snprintf(text, sizeof(text), "%.9g", static_cast<double>(row.probability));
            events.push_back("{\"event\":\"token\",\"request_id\":\"" + wire_detail::escape(request.request_id) + "\",\"session_id\":\"" +
                             wire_detail::escape(request.session_id) + "\",\"index\":" + std::to_string(request.generated) +
                             ",\"token_id\":" + std::to_string(row.token_id) + ",\"probability\":" + text +
                             ",\"is_stop_token\":" + (is_stop ? "true" : "false") + "}");
            ++request.generated;
            // the stop token is emitted, then the generation ends (session.cpp:1008-1012)
            if (is_stop || request.generated >= request.max_new_tokens)
                events.push_back(done_event(request, is_stop));
            else
                still_active.push_back(std::move(request));
        }
        active_ = std::move(still_active);
        return events;
    }

private:
    struct SessionEntry
    {
        std::string id;
        uint64_t seed = 0;
        uint64_t uniforms_drawn = 0;
    };

    WireSamplingRouter(detail::Handle handle, uint32_t max_sessions) : handle_(std::move(handle)), max_sessions_(max_sessions) {}

    // validate_sampling_options (session.cpp:65-74), same order
    static int validate(const moe_row_params& p)
    {
        const bool t_ok = (p.temperature == p.temperature) && (p.temperature - p.temperature == 0.0f) && p.temperature >= 0.0f;
        if (!t_ok)
            return MOE_ROW_BAD_TEMPERATURE;
        if (!((p.top_p - p.top_p == 0.0f) && p.top_p > 0.0f && p.top_p <= 1.0f))
            return MOE_ROW_BAD_TOP_P;
        if (!((p.min_p - p.min_p == 0.0f) && p.min_p >= 0.0f && p.min_p <= 1.0f))
            return MOE_ROW_BAD_MIN_P;
        return MOE_ROW_OK;
    }

    size_t find_session(std::string_view id) const
    {
        for (size_t i = 0; i < sessions_.size(); ++i)
            if (sessions_[i].id == id)
                return i;
        return sessions_.size();
    }

    static std::string done_event(const ActiveRequest& request, bool stopped_by_stop_token)
    {
        return "{\"event\":\"done\",\"request_id\":\"" + wire_detail::escape(request.request_id) + "\",\"session_id\":\"" +
               wire_detail::escape(request.session_id) + "\",\"ok\":true,\"generated_tokens\":" + std::to_string(request.generated) +
               ",\"stopped_by_stop_token\":" + (stopped_by_stop_token ? "true" : "false") + ",\"stopped_by_callback\":" +
               (request.cancelled ? "true" : "false") + ",\"cancelled\":" + (request.cancelled ? "true" : "false") + "}";
    }

    void retire_cancelled(std::vector<std::string>& events)
    {
        std::vector<ActiveRequest> kept;
        for (ActiveRequest& request : active_)
        {
            if (request.cancelled)
                events.push_back(done_event(request, false));
            else
                kept.push_back(std::move(request));
        }
        active_ = std::move(kept);
    }

    detail::Handle handle_;
    uint32_t max_sessions_ = 0;
    std::vector<SessionEntry> sessions_;
    std::vector<ActiveRequest> active_;
    std::vector<moe_row_params> params_;
    std::vector<int32_t> stop_offsets_, stop_tokens_;
    moe_sampled_row* sampled_rows_ = nullptr;
};

} // namespace moe_b200
