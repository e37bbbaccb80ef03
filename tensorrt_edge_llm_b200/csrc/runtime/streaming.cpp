#include "streaming.h"

namespace telb {

const char* to_string(FinishReason r) {
    switch (r) {
        case FinishReason::kNotFinished: return "not_finished";
        case FinishReason::kEndId: return "stop";
        case FinishReason::kLength: return "length";
        case FinishReason::kCancelled: return "cancelled";
        case FinishReason::kError: return "error";
        case FinishReason::kStopWords: return "stop_words";
    }
    return "unknown";
}

void StreamChannel::flush_locked(bool force) {
    if (pending_.empty() && !force) return;
    if (!force && static_cast<int>(pending_.size()) < interval_) return;
    StreamChunk c;
    c.token_ids.swap(pending_);
    std::swap(c.logprobs, pending_lp_);
    q_.push_back(std::move(c));
}

void StreamChannel::push(const std::vector<int32_t>& tokens, const TokenLogprobs& logprobs) {
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (finished_) return;
        const auto now = std::chrono::steady_clock::now();
        if (generated_ == 0 && !tokens.empty()) t_first_ = now;
        t_last_ = now;
        generated_ += static_cast<int>(tokens.size());
        pending_.insert(pending_.end(), tokens.begin(), tokens.end());
        pending_lp_.append(logprobs);
        flush_locked(false);
    }
    cv_.notify_all();
}

void StreamChannel::finish(FinishReason reason) {
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (finished_) return;
        finished_ = true;
        reason_ = reason;
        StreamChunk c;
        c.token_ids.swap(pending_);
        std::swap(c.logprobs, pending_lp_);
        c.finished = true;
        c.reason = reason;
        q_.push_back(std::move(c));
    }
    cv_.notify_all();
}

bool StreamChannel::try_pop(StreamChunk& out) {
    std::lock_guard<std::mutex> lk(mu_);
    if (q_.empty()) return false;
    out = std::move(q_.front());
    q_.pop_front();
    return true;
}

bool StreamChannel::wait_pop(StreamChunk& out, double timeout_s) {
    std::unique_lock<std::mutex> lk(mu_);
    if (!cv_.wait_for(lk, std::chrono::duration<double>(timeout_s), [&] { return !q_.empty(); })) return false;
    out = std::move(q_.front());
    q_.pop_front();
    return true;
}

void StreamChannel::cancel() { cancelled_.store(true); }

bool StreamChannel::is_finished() const {
    std::lock_guard<std::mutex> lk(mu_);
    return finished_;
}

FinishReason StreamChannel::reason() const {
    std::lock_guard<std::mutex> lk(mu_);
    return reason_;
}

GenerationMetrics StreamChannel::metrics() const {
    std::lock_guard<std::mutex> lk(mu_);
    GenerationMetrics m;
    m.generated_tokens = generated_;
    if (collect_ && generated_ > 0) {
        m.time_to_first_token_s = std::chrono::duration<double>(t_first_ - t0_).count();
        m.generation_time_s = std::chrono::duration<double>(t_last_ - t_first_).count();
    }
    return m;
}

size_t utf8_complete_prefix(const std::string& s) {
    const size_t n = s.size();
    size_t i = n;
    int back = 0;
    while (i > 0 && back < 4) {
        const unsigned char c = static_cast<unsigned char>(s[i - 1]);
        if ((c & 0xC0) == 0x80) {       // continuation byte: keep walking back
            --i;
            ++back;
            continue;
        }
        int need = 0;
        if (c >= 0xF0) need = 3;
        else if (c >= 0xE0) need = 2;
        else if (c >= 0xC0) need = 1;
        if (back < need) return i - 1;  // the last lead byte is missing continuation bytes
        return n;
    }
    return back == 0 ? n : i;
}

}  // namespace telb
