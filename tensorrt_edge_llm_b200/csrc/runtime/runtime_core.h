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
    // ---- the rest of what a prepared model's runtime_config.json records (`from_runtime_config`) ----
    int intermediate_size = 0, max_position_embeddings = 0, rotary_dim = 0;
    double rms_norm_eps = 1e-6, rope_theta = 10000.0, rope_scaling_factor = 1.0, final_logit_softcapping = 0.0;
    std::string rope_scaling_type;                 // "", linear, dynamic, llama3, yarn, longrope
    std::vector<int> mrope_section;                // multimodal RoPE: rotary pairs per (t, h, w) component
    bool has_qk_norm = false, attention_bias = false, attention_sink_bias = false, attention_k_eq_v = false, has_value_norm = false;
    int sliding_window = 0;                        // 0 = none
    std::vector<int> layer_windows;                // per layer (empty = sliding_window everywhere)
    std::vector<std::string> layer_types;          // attention / mamba / gdn / none per layer
    std::vector<std::string> mlp_types;            // mlp / moe / none per layer
    int num_kv_shared_layers = 0;
    int num_experts = 0, num_experts_per_tok = 0, moe_intermediate_size = 0, shared_expert_intermediate_size = 0;
    std::string router_type;
    int quant_group_size = 0;
    std::string lm_head_quantization;
    // recurrent mixers (0 when the model has none)
    int mamba_num_heads = 0, mamba_head_dim = 0, mamba_d_state = 0, mamba_n_groups = 0, mamba_conv_kernel = 0;
    int gdn_num_k_heads = 0, gdn_num_v_heads = 0, gdn_head_k_dim = 0, gdn_head_v_dim = 0, gdn_conv_kernel = 0;
    // draft heads
    std::string draft_type, dflash_projector_type;
    int draft_vocab_size = 0, eagle3_num_target_layers = 0, dflash_block_size = 0, dflash_version = 1, dflash_mask_token_id = 0;
    int draft_candidate_count = 0, dspark_markov_rank = 0;
    bool eagle_fc_norm = false, eagle_norm_output = false, dspark_enable_confidence_head = false;
    // block diffusion
    bool is_diffusion = false;
    int diffusion_canvas_length = 0, diffusion_max_steps = 0;
    std::vector<int> eos_token_ids;
    int bos_token_id = -1;

    static LLMEngineConfig from_json(const Json& j);
    // From the `runtime_config.json` of a prepared model ({"model": {...}, "deployment": {...}}).
    static LLMEngineConfig from_runtime_config(const Json& j);
    Json to_json() const;
    // Derived quantities.
    bool is_hybrid() const;
    bool is_moe() const { return num_experts > 0; }
    int num_attention_layers() const;              // layers that own a KV cache (KV-shared layers excluded)
    int num_recurrent_layers() const;
    long long kv_bytes_per_token() const;          // every KV-owning layer, K and V, at the cache's element size
    long long kv_pool_bytes() const;               // max_batch_size sequences of max_kv_cache_capacity tokens, whole pages
    long long recurrent_state_bytes_per_seat() const;
    // Empty when the configuration is consistent, else the first problem found.
    std::string validate() const;
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
