// Smaller runtime services: ragged batch builder, host sampler, engine / parallel configuration,
// LoRA registry, sticky device-failure state, logger and stage timer.
//
// Counterparts in the reference: cpp/runtime/exec/raggedBatchBuilder.{h,cpp} and scheduledStep.h,
// cpp/sampler/sampling.h:36-160 (RowSamplingParams, greedy rule, per-row uniforms, default seed 42),
// cpp/runtime/config/llmEngineConfig.{h,cpp}, cpp/runtime/multiDevice/parallelConfig.h,
// cpp/runtime/state/loraManager.{h,cpp}, cpp/runtime/deviceFailure.h:33-60, cpp/common/logger.h
// (EDGELLM_LOG_LEVEL), cpp/profiling/{timer,metrics}.h.
#pragma once

#include <chrono>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "json.h"
#include "scheduler.h"

namespace telb {

// ---- ragged batch -------------------------------------------------------------------------------
// Flattened metadata of one step, ready to be copied to the device in one transfer.
struct RaggedBatch {
    std::vector<int32_t> q_start, q_len, past_len, positions, seq_ids, slot_ids, logits_idx;
    int num_seqs = 0, num_tokens = 0, max_q_len = 0, max_seq_len = 0;
};

class RaggedBatchBuilder {
  public:
    // `past_lens[i]` = tokens already cached for plan.seqs[i]; logits are requested for decode rows
    // and for context chunks that complete their prompt.
    static RaggedBatch build(const StepPlan& plan, const std::vector<int>& past_lens, bool logits_all = false);
};

// ---- sampling (host reference; the device kernels implement the same rules) -----------------------
struct RowSamplingParams {
    float temperature = 0.f;
    int top_k = 0;
    float top_p = 1.f;
    bool greedy() const { return temperature < 1e-3f; }
    bool use_top_k() const { return top_k > 0; }
    bool use_top_p() const { return top_p < 1.f || top_k <= 0; }
};
// Counter-based uniform in [0,1): depends only on (seed, request, step), never on batch position.
float request_stable_uniform(uint64_t seed, uint64_t request_id, uint64_t step);
int32_t sample_row(const float* logits, int vocab, const RowSamplingParams& p, float uniform);
void apply_token_bitmask(float* logits, int vocab, const int32_t* bitmask_words);
constexpr float kMaskedLogitValue = -1e30f;

// ---- configuration ------------------------------------------------------------------------------
enum class ParallelType { kTensor = 0, kExpert = 1 };
struct ParallelConfig {
    ParallelType type = ParallelType::kTensor;
    int world_size = 1, rank = 0;
    std::string launch_mode = "process";       // one process per GPU (torch.distributed)
    std::string validate() const;
};

// Keys of the runtime `config.json` written by the build step.
struct LLMEngineConfig {
    std::string model_type = "llama";
    int vocab_size = 0, hidden_size = 0, num_layers = 0, num_heads = 0, num_kv_heads = 0, head_dim = 0;
    int max_batch_size = 1, max_input_len = 2048, max_kv_cache_capacity = 4096, kv_page_size = 64;
    std::string dtype = "bfloat16", quantization = "fp16", kv_cache_dtype = "auto";
    std::vector<std::string> decoding_strategies = {"vanilla"};
    int world_size = 1;
    static LLMEngineConfig from_json(const Json& j);
    Json to_json() const;
};

// ---- LoRA registry ------------------------------------------------------------------------------
struct LoraAdapter {
    std::string name, path;
    int rank = 0;
    float scale = 1.f;
};
class LoRAManager {
  public:
    void add(const LoraAdapter& a);
    bool remove(const std::string& name);
    const LoraAdapter* find(const std::string& name) const;
    bool activate(const std::string& name);            // O(1): only the active index changes
    const LoraAdapter* active() const;
    std::vector<std::string> names() const;

  private:
    std::map<std::string, LoraAdapter> adapters_;
    std::string active_;
};

// ---- failure state ------------------------------------------------------------------------------
class DeviceFailureState {
  public:
    void record(const std::string& what);
    bool failed() const;
    std::string reason() const;

  private:
    mutable std::mutex mu_;
    bool failed_ = false;
    std::string reason_;
};

// ---- logging / profiling ------------------------------------------------------------------------
enum class LogLevel { kVerbose = 0, kInfo, kWarning, kError, kNone };
LogLevel log_level_from_env();                          // EDGELLM_LOG_LEVEL = VERBOSE|INFO|WARNING|ERROR|NONE
void log_message(LogLevel lvl, const std::string& msg);

class StageTimer {
  public:
    void set_enabled(bool on) { enabled_ = on; }
    void begin(const std::string& stage);
    void end(const std::string& stage);
    struct Sample {
        uint64_t count = 0;
        double total_s = 0.0, max_s = 0.0;
    };
    std::map<std::string, Sample> snapshot() const;
    void reset();

  private:
    bool enabled_ = true;
    mutable std::mutex mu_;
    std::map<std::string, std::chrono::steady_clock::time_point> open_;
    std::map<std::string, Sample> samples_;
};

}  // namespace telb
