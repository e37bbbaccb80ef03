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

LLMEngineConfig LLMEngineConfig::from_runtime_config(const Json& root) {
    const Json& m = root["model"].is_object() ? root["model"] : root;
    LLMEngineConfig c = from_json(m);
    const Json& d = root["deployment"];
    auto di = [&](const char* k, int& dst) { if (d.is_object() && d[k].is_number()) dst = static_cast<int>(d[k].as_int()); };
    di("max_batch_size", c.max_batch_size);
    di("max_input_len", c.max_input_len);
    di("max_kv_cache_capacity", c.max_kv_cache_capacity);
    di("kv_page_size", c.kv_page_size);
    di("tensor_parallel_size", c.world_size);
    auto i = [&](const Json& j, const char* k, int& dst) { if (j.is_object() && j[k].is_number()) dst = static_cast<int>(j[k].as_int()); };
    auto f = [&](const Json& j, const char* k, double& dst) { if (j.is_object() && j[k].is_number()) dst = j[k].as_double(); };
    auto b = [&](const Json& j, const char* k, bool& dst) { if (j.is_object() && j[k].is_bool()) dst = j[k].as_bool(); };
    auto s = [&](const Json& j, const char* k, std::string& dst) { if (j.is_object() && j[k].is_string()) dst = j[k].as_string(); };
    auto vi = [&](const Json& j, const char* k, std::vector<int>& dst) {
        if (j.is_object() && j[k].is_array()) {
            dst.clear();
            for (const auto& v : j[k].items()) dst.push_back(static_cast<int>(v.as_int()));
        }
    };
    auto vs = [&](const Json& j, const char* k, std::vector<std::string>& dst) {
        if (j.is_object() && j[k].is_array()) {
            dst.clear();
            for (const auto& v : j[k].items()) dst.push_back(v.is_string() ? v.as_string() : std::string());
        }
    };
    i(m, "intermediate_size", c.intermediate_size);
    i(m, "max_position_embeddings", c.max_position_embeddings);
    f(m, "rms_norm_eps", c.rms_norm_eps);
    f(m, "rope_theta", c.rope_theta);
    f(m, "final_logit_softcapping", c.final_logit_softcapping);
    double partial = 1.0;
    f(m, "partial_rotary_factor", partial);
    c.rotary_dim = static_cast<int>(c.head_dim * partial + 0.5) & ~1;
    const Json& rs = m["rope_scaling"];
    if (rs.is_object()) {
        s(rs, "rope_type", c.rope_scaling_type);
        if (c.rope_scaling_type.empty()) s(rs, "type", c.rope_scaling_type);
        f(rs, "factor", c.rope_scaling_factor);
    }
    vi(m, "mrope_section", c.mrope_section);
    b(m, "has_qk_norm", c.has_qk_norm);
    b(m, "attention_bias", c.attention_bias);
    b(m, "attention_sink_bias", c.attention_sink_bias);
    b(m, "attention_k_eq_v", c.attention_k_eq_v);
    b(m, "has_value_norm", c.has_value_norm);
    i(m, "sliding_window", c.sliding_window);
    vi(m, "layer_windows", c.layer_windows);
    vs(m, "layer_types", c.layer_types);
    vs(m, "mlp_types", c.mlp_types);
    i(m, "num_kv_shared_layers", c.num_kv_shared_layers);
    i(m, "num_experts", c.num_experts);
    i(m, "num_experts_per_tok", c.num_experts_per_tok);
    i(m, "moe_intermediate_size", c.moe_intermediate_size);
    i(m, "shared_expert_intermediate_size", c.shared_expert_intermediate_size);
    s(m, "router_type", c.router_type);
    const Json& q = m["quant"];
    if (q.is_object()) {
        s(q, "quant_type", c.quantization);
        i(q, "group_size", c.quant_group_size);
        s(q, "lm_head_quant_type", c.lm_head_quantization);
        std::string kvq;
        s(q, "kv_cache_quant", kvq);
        if (!kvq.empty()) c.kv_cache_dtype = kvq;
    }
    const Json& mb = m["mamba"];
    i(mb, "num_heads", c.mamba_num_heads);
    i(mb, "head_dim", c.mamba_head_dim);
    i(mb, "d_state", c.mamba_d_state);
    i(mb, "n_groups", c.mamba_n_groups);
    i(mb, "conv_kernel", c.mamba_conv_kernel);
    const Json& gd = m["gdn"];
    i(gd, "num_k_heads", c.gdn_num_k_heads);
    i(gd, "num_v_heads", c.gdn_num_v_heads);
    i(gd, "head_k_dim", c.gdn_head_k_dim);
    i(gd, "head_v_dim", c.gdn_head_v_dim);
    i(gd, "conv_kernel", c.gdn_conv_kernel);
    s(m, "draft_type", c.draft_type);
    s(m, "dflash_projector_type", c.dflash_projector_type);
    i(m, "draft_vocab_size", c.draft_vocab_size);
    i(m, "eagle3_num_target_layers", c.eagle3_num_target_layers);
    i(m, "dflash_block_size", c.dflash_block_size);
    i(m, "dflash_version", c.dflash_version);
    i(m, "dflash_mask_token_id", c.dflash_mask_token_id);
    i(m, "draft_candidate_count", c.draft_candidate_count);
    i(m, "dspark_markov_rank", c.dspark_markov_rank);
    b(m, "eagle_fc_norm", c.eagle_fc_norm);
    b(m, "eagle_norm_output", c.eagle_norm_output);
    b(m, "dspark_enable_confidence_head", c.dspark_enable_confidence_head);
    const Json& df = m["diffusion"];
    if (df.is_object()) {
        c.is_diffusion = true;
        i(df, "canvas_length", c.diffusion_canvas_length);
        i(df, "max_denoising_steps", c.diffusion_max_steps);
    }
    i(m, "bos_token_id", c.bos_token_id);
    if (m["eos_token_id"].is_number()) c.eos_token_ids = {static_cast<int>(m["eos_token_id"].as_int())};
    else vi(m, "eos_token_id", c.eos_token_ids);
    c.decoding_strategies = {"vanilla"};
    if (c.is_diffusion) c.decoding_strategies = {"block_diffusion"};
    return c;
}

bool LLMEngineConfig::is_hybrid() const {
    for (const auto& t : layer_types)
        if (t != "attention") return true;
    return false;
}

int LLMEngineConfig::num_recurrent_layers() const {
    int n = 0;
    for (const auto& t : layer_types) n += (t == "mamba" || t == "gdn") ? 1 : 0;
    return n;
}

int LLMEngineConfig::num_attention_layers() const {
    int n = 0;
    if (layer_types.empty()) n = num_layers;
    else
        for (const auto& t : layer_types) n += t == "attention" ? 1 : 0;
    return std::max(0, n - num_kv_shared_layers);
}

static int element_bytes(const std::string& dtype) { return dtype == "float32" ? 4 : ((dtype == "fp8" || dtype == "FP8") ? 1 : 2); }

long long LLMEngineConfig::kv_bytes_per_token() const {
    const int eb = (kv_cache_dtype == "auto" || kv_cache_dtype.empty() || kv_cache_dtype == "model") ? element_bytes(dtype) : element_bytes(kv_cache_dtype);
    const int kvh = std::max(1, num_kv_heads / std::max(1, world_size));
    return 2LL * num_attention_layers() * kvh * head_dim * eb;
}

long long LLMEngineConfig::kv_pool_bytes() const {
    const long long pages_per_seq = (max_kv_cache_capacity + kv_page_size - 1) / std::max(1, kv_page_size);
    return kv_bytes_per_token() * kv_page_size * (pages_per_seq * max_batch_size + 1);
}

long long LLMEngineConfig::recurrent_state_bytes_per_seat() const {
    long long total = 0;
    const int eb = element_bytes(dtype), tp = std::max(1, world_size);
    for (const auto& t : layer_types) {
        if (t == "mamba") {
            const long long inner = 1LL * mamba_num_heads * mamba_head_dim;
            total += (inner + 2LL * mamba_n_groups * mamba_d_state) / tp * (mamba_conv_kernel - 1) * eb;      // convolution window
            total += 1LL * mamba_num_heads / tp * mamba_head_dim * mamba_d_state * 4;                         // fp32 SSM state
        } else if (t == "gdn") {
            total += (2LL * gdn_num_k_heads * gdn_head_k_dim + 1LL * gdn_num_v_heads * gdn_head_v_dim) / tp * (gdn_conv_kernel - 1) * eb;
            total += 1LL * gdn_num_v_heads / tp * gdn_head_k_dim * gdn_head_v_dim * 4;
        }
    }
    return total;
}

std::string LLMEngineConfig::validate() const {
    if (vocab_size <= 0 || hidden_size <= 0 || num_layers <= 0) return "vocab_size, hidden_size and num_hidden_layers must be positive";
    if (num_heads <= 0 || head_dim <= 0) return "num_attention_heads and head_dim must be positive";
    if (num_kv_heads <= 0 || num_heads % num_kv_heads) return "num_attention_heads must be a multiple of num_key_value_heads";
    if (!layer_types.empty() && static_cast<int>(layer_types.size()) != num_layers) return "layer_types needs one entry per layer";
    if (!layer_windows.empty() && static_cast<int>(layer_windows.size()) != num_layers) return "layer_windows needs one entry per layer";
    if (kv_page_size != 64 && kv_page_size != 128 && kv_page_size != 16 && kv_page_size != 32) return "kv_page_size must be 16, 32, 64 or 128";
    if (max_batch_size <= 0 || max_input_len <= 0 || max_kv_cache_capacity < max_input_len) return "deployment limits: max_kv_cache_capacity must hold max_input_len";
    if (world_size > 1 && (num_heads % world_size)) return "num_attention_heads must divide over the tensor-parallel ranks";
    if (num_kv_shared_layers < 0 || num_kv_shared_layers >= num_layers) return "num_kv_shared_layers must leave a layer with its own cache";
    if (num_experts > 0 && (num_experts_per_tok <= 0 || num_experts_per_tok > num_experts)) return "num_experts_per_tok must be in 1..num_experts";
    for (const auto& t : layer_types) {
        if (t == "mamba" && (mamba_num_heads <= 0 || mamba_d_state <= 0)) return "a mamba layer needs the mamba section";
        if (t == "gdn" && (gdn_num_v_heads <= 0 || gdn_head_k_dim <= 0)) return "a gdn layer needs the gdn section";
    }
    if (draft_type == "dflash" && dflash_block_size < 2) return "a block draft needs dflash_block_size >= 2";
    return std::string();
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
