#include "runtime_core.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <numeric>

namespace telb {

RaggedBatch RaggedBatchBuilder::build(const StepPlan& plan, const std::vector<int>& past_lens, bool logits_all) {
    RaggedBatch b;
    b.num_seqs = static_cast<int>(plan.seqs.size());
    b.q_start.push_back(0);
    for (int i = 0; i < b.num_seqs; ++i) {
        const PlannedSequence& s = plan.seqs[i];
        const int past = past_lens.at(i);
        b.q_len.push_back(s.length);
        b.past_len.push_back(past);
        b.slot_ids.push_back(s.slot);
        for (int t = 0; t < s.length; ++t) {
            b.positions.push_back(past + t);
            b.seq_ids.push_back(i);
            if (logits_all) b.logits_idx.push_back(b.num_tokens + t);
        }
        b.num_tokens += s.length;
        b.q_start.push_back(b.num_tokens);
        if (!logits_all && (s.kind == WorkKind::kDecode || s.last_chunk)) b.logits_idx.push_back(b.num_tokens - 1);
        b.max_q_len = std::max(b.max_q_len, s.length);
        b.max_seq_len = std::max(b.max_seq_len, past + s.length);
    }
    return b;
}

// splitmix64-based counter RNG
static uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

float request_stable_uniform(uint64_t seed, uint64_t request_id, uint64_t step) {
    const uint64_t h = mix64(mix64(mix64(seed) ^ request_id) ^ step);
    return static_cast<float>((h >> 40) * (1.0 / 16777216.0));      // 24 random bits
}

int32_t sample_row(const float* logits, int vocab, const RowSamplingParams& p, float uniform) {
    if (p.greedy()) return static_cast<int32_t>(std::max_element(logits, logits + vocab) - logits);
    std::vector<int32_t> idx(vocab);
    std::iota(idx.begin(), idx.end(), 0);
    const int k = p.use_top_k() ? std::min(p.top_k, vocab) : vocab;
    std::partial_sort(idx.begin(), idx.begin() + k, idx.end(), [&](int32_t a, int32_t b) {
        return logits[a] > logits[b] || (logits[a] == logits[b] && a < b);
    });
    std::vector<double> prob(k);
    const double mx = logits[idx[0]] / p.temperature;
    double sum = 0;
    for (int i = 0; i < k; ++i) sum += (prob[i] = std::exp(logits[idx[i]] / p.temperature - mx));
    for (auto& q : prob) q /= sum;
    int keep = k;
    if (p.top_p < 1.f) {
        double cum = 0;
        for (int i = 0; i < k; ++i) {
            if (cum >= p.top_p) { keep = i; break; }
            cum += prob[i];
        }
        keep = std::max(keep, 1);
    }
    double tot = 0;
    for (int i = 0; i < keep; ++i) tot += prob[i];
    const double target = uniform * tot;
    double cum = 0;
    for (int i = 0; i < keep; ++i) {
        cum += prob[i];
        if (target < cum) return idx[i];
    }
    return idx[keep - 1];
}

void apply_token_bitmask(float* logits, int vocab, const int32_t* words) {
    for (int i = 0; i < vocab; ++i)
        if (!((words[i >> 5] >> (i & 31)) & 1)) logits[i] = kMaskedLogitValue;
}

std::string ParallelConfig::validate() const {
    if (world_size < 1) return "world_size must be positive";
    if (rank < 0 || rank >= world_size) return "rank outside [0, world_size)";
    if (world_size > 8) return "a single node holds at most 8 ranks";
    return "";
}

LLMEngineConfig LLMEngineConfig::from_json(const Json& j) {
    LLMEngineConfig c;
    auto s = [&](const char* k, std::string& dst) { if (j[k].is_string()) dst = j[k].as_string(); };
    auto i = [&](const char* k, int& dst) { if (j[k].is_number()) dst = static_cast<int>(j[k].as_int()); };
    s("model_type", c.model_type);
    i("vocab_size", c.vocab_size);
    i("hidden_size", c.hidden_size);
    i("num_hidden_layers", c.num_layers);
    i("num_attention_heads", c.num_heads);
    i("num_key_value_heads", c.num_kv_heads);
    i("head_dim", c.head_dim);
    i("max_batch_size", c.max_batch_size);
    i("max_input_len", c.max_input_len);
    i("max_kv_cache_capacity", c.max_kv_cache_capacity);
    i("kv_page_size", c.kv_page_size);
    i("world_size", c.world_size);
    s("dtype", c.dtype);
    s("quantization", c.quantization);
    s("kv_cache_dtype", c.kv_cache_dtype);
    if (j["decoding_strategies"].is_array()) {
        c.decoding_strategies.clear();
        for (const auto& v : j["decoding_strategies"].items()) c.decoding_strategies.push_back(v.as_string());
    }
    if (c.head_dim == 0 && c.num_heads > 0) c.head_dim = c.hidden_size / c.num_heads;
    if (c.num_kv_heads == 0) c.num_kv_heads = c.num_heads;
    return c;
}

Json LLMEngineConfig::to_json() const {
    Json j = Json::object();
    j.set("model_type", model_type);
    j.set("vocab_size", vocab_size);
    j.set("hidden_size", hidden_size);
    j.set("num_hidden_layers", num_layers);
    j.set("num_attention_heads", num_heads);
    j.set("num_key_value_heads", num_kv_heads);
    j.set("head_dim", head_dim);
    j.set("max_batch_size", max_batch_size);
    j.set("max_input_len", max_input_len);
    j.set("max_kv_cache_capacity", max_kv_cache_capacity);
    j.set("kv_page_size", kv_page_size);
    j.set("world_size", world_size);
    j.set("dtype", dtype);
    j.set("quantization", quantization);
    j.set("kv_cache_dtype", kv_cache_dtype);
    Json arr = Json::array();
    for (const auto& s : decoding_strategies) arr.push_back(Json(s));
    j.set("decoding_strategies", arr);
    return j;
}

void LoRAManager::add(const LoraAdapter& a) { adapters_[a.name] = a; }
bool LoRAManager::remove(const std::string& name) {
    if (active_ == name) active_.clear();
    return adapters_.erase(name) > 0;
}
const LoraAdapter* LoRAManager::find(const std::string& name) const {
    auto it = adapters_.find(name);
    return it == adapters_.end() ? nullptr : &it->second;
}
bool LoRAManager::activate(const std::string& name) {
    if (name.empty()) { active_.clear(); return true; }
    if (!adapters_.count(name)) return false;
    active_ = name;
    return true;
}
const LoraAdapter* LoRAManager::active() const { return active_.empty() ? nullptr : find(active_); }
std::vector<std::string> LoRAManager::names() const {
    std::vector<std::string> out;
    for (const auto& kv : adapters_) out.push_back(kv.first);
    return out;
}

void DeviceFailureState::record(const std::string& what) {
    std::lock_guard<std::mutex> lk(mu_);
    if (!failed_) { failed_ = true; reason_ = what; }      // sticky: the first failure is kept
}
bool DeviceFailureState::failed() const { std::lock_guard<std::mutex> lk(mu_); return failed_; }
std::string DeviceFailureState::reason() const { std::lock_guard<std::mutex> lk(mu_); return reason_; }

LogLevel log_level_from_env() {
    const char* e = std::getenv("EDGELLM_LOG_LEVEL");
    if (!e) return LogLevel::kWarning;
    std::string s(e);
    std::transform(s.begin(), s.end(), s.begin(), ::toupper);
    if (s == "VERBOSE" || s == "DEBUG") return LogLevel::kVerbose;
    if (s == "INFO") return LogLevel::kInfo;
    if (s == "WARNING" || s == "WARN") return LogLevel::kWarning;
    if (s == "ERROR") return LogLevel::kError;
    if (s == "NONE" || s == "OFF") return LogLevel::kNone;
    return LogLevel::kWarning;
}

void log_message(LogLevel lvl, const std::string& msg) {
    static const LogLevel floor = log_level_from_env();
    if (lvl < floor) return;
    static const char* names[] = {"VERBOSE", "INFO", "WARNING", "ERROR", "NONE"};
    fprintf(stderr, "[telb][%s] %s\n", names[static_cast<int>(lvl)], msg.c_str());
}

void StageTimer::begin(const std::string& stage) {
    if (!enabled_) return;
    std::lock_guard<std::mutex> lk(mu_);
    open_[stage] = std::chrono::steady_clock::now();
}
void StageTimer::end(const std::string& stage) {
    if (!enabled_) return;
    const auto now = std::chrono::steady_clock::now();
    std::lock_guard<std::mutex> lk(mu_);
    auto it = open_.find(stage);
    if (it == open_.end()) return;
    const double dt = std::chrono::duration<double>(now - it->second).count();
    open_.erase(it);
    Sample& s = samples_[stage];
    ++s.count;
    s.total_s += dt;
    s.max_s = std::max(s.max_s, dt);
}
std::map<std::string, StageTimer::Sample> StageTimer::snapshot() const {
    std::lock_guard<std::mutex> lk(mu_);
    return samples_;
}
void StageTimer::reset() {
    std::lock_guard<std::mutex> lk(mu_);
    samples_.clear();
    open_.clear();
}

}  // namespace telb
