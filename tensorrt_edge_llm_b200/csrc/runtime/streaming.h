// Token streaming between the engine's actor thread and consumer threads.
//
// Counterpart of cpp/runtime/streaming.{h,cpp} in the reference (FinishReason, StreamChunk,
// StreamChannel with mutex + condition variable + deque, cancel, stream interval) and the design
// note docs/source/developer_guide/software-design/llm-streaming.md.
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace telb {

enum class FinishReason { kNotFinished = 0, kEndId, kLength, kCancelled, kError, kStopWords };
const char* to_string(FinishReason r);

// Log-probabilities that travel with generated tokens: `chosen[i]` belongs to token i; when the request
// asked for the k most likely alternatives, `top_ids` / `top_values` hold k entries per token.
struct TokenLogprobs {
    std::vector<float> chosen;
    std::vector<int32_t> top_ids;
    std::vector<float> top_values;
    bool empty() const { return chosen.empty(); }
    void append(const TokenLogprobs& o) {
        chosen.insert(chosen.end(), o.chosen.begin(), o.chosen.end());
        top_ids.insert(top_ids.end(), o.top_ids.begin(), o.top_ids.end());
        top_values.insert(top_values.end(), o.top_values.begin(), o.top_values.end());
    }
};

struct StreamChunk {
    std::vector<int32_t> token_ids;
    TokenLogprobs logprobs;
    std::string text;            // filled by a detokenising consumer, empty otherwise
    bool finished = false;
    FinishReason reason = FinishReason::kNotFinished;
};

struct GenerationMetrics {
    int generated_tokens = 0;
    double time_to_first_token_s = 0.0;
    double generation_time_s = 0.0;          // first token → last token
    double decode_tokens_per_second() const {
        return (generated_tokens > 1 && generation_time_s > 0) ? (generated_tokens - 1) / generation_time_s : 0.0;
    }
};

class StreamChannel {
  public:
    static std::shared_ptr<StreamChannel> create(bool collect_metrics = false) {
        return std::shared_ptr<StreamChannel>(new StreamChannel(collect_metrics));
    }
    // producer side (actor thread)
    void push(const std::vector<int32_t>& tokens, const TokenLogprobs& logprobs = TokenLogprobs());
    void finish(FinishReason reason);
    // consumer side
    bool try_pop(StreamChunk& out);
    bool wait_pop(StreamChunk& out, double timeout_s);      // false on timeout
    void cancel();                                          // consumer went away; engine frees the seat at its next boundary
    bool cancelled() const { return cancelled_.load(); }
    bool is_finished() const;
    FinishReason reason() const;
    void set_stream_interval(int n) { interval_ = n < 1 ? 1 : n; }
    GenerationMetrics metrics() const;

  private:
    explicit StreamChannel(bool collect) : collect_(collect), t0_(std::chrono::steady_clock::now()) {}
    void flush_locked(bool force);
    mutable std::mutex mu_;
    std::condition_variable cv_;
    std::deque<StreamChunk> q_;
    std::vector<int32_t> pending_;
    TokenLogprobs pending_lp_;
    std::atomic<bool> cancelled_{false};
    bool finished_ = false;
    FinishReason reason_ = FinishReason::kNotFinished;
    int interval_ = 1;
    bool collect_;
    std::chrono::steady_clock::time_point t0_, t_first_, t_last_;
    int generated_ = 0;
};

// Incremental UTF-8 boundary tracking: returns how many leading bytes of `bytes` form complete
// code points, so a streamed detokenisation never emits half a character.
size_t utf8_complete_prefix(const std::string& bytes);

}  // namespace telb
