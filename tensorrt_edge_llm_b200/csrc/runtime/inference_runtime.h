// The runtime façade: one object that turns a batch of chat conversations / prompts into generated text.
//
// It owns the request engine (scheduler.h) and borrows a tokenizer and a chat template.  handle_request() renders and
// tokenises every entry, submits them all (the engine batches them in flight with whatever else is resident), drains their
// stream channels, detokenises incrementally on UTF-8 boundaries, applies textual stop sequences and returns ids, text,
// finish reasons and per-request timings.  Clients that bring their own token ids and want a handle back use submit()
// ("seated admission"); clients that want to drive the model step by step open a session of their own through
// open_session() ("stepped execution").  The model itself sits behind the RuntimeSession seam, so the façade is the same
// for the GPU runner and for a scripted session in tests.
//
// Counterpart of cpp/runtime/llmInferenceRuntime.h (handleRequest, captureDecodingCUDAGraph, openSession,
// unavailableReason, hasDraftModel, supportsSeatedAdmission / supportsSteppedExecution) in the reference.
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "scheduler.h"
#include "tokenizer.h"

namespace telb {

struct RuntimeOptions {
    EngineConfig engine;
    bool has_draft_model = false;
    // Warm-up hook (CUDA-graph capture of the decode step on the GPU runner).  Called by capture_decoding_cuda_graph() only
    // while nothing is queued or resident; null = nothing to capture.
    std::function<bool()> capture_hook;
};

struct LLMGenerationRequest {
    struct Entry {
        std::vector<ChatMessage> messages;      // rendered with the chat template ...
        std::string prompt;                     // ... or a plain prompt ...
        std::vector<int32_t> prompt_ids;        // ... or ready token ids (first non-empty of ids, messages, prompt wins)
    };
    std::vector<Entry> requests;
    int max_generate_length = 128;
    float temperature = 0.f;                    // 0 = greedy
    int top_k = 0;
    float top_p = 1.f;
    uint64_t seed = 42;
    bool apply_chat_template = true;
    bool add_generation_prompt = true;
    bool enable_thinking = true;
    bool ignore_eos = false;
    std::vector<std::string> stop;              // textual stop sequences: generation ends before the first occurrence
    std::vector<int32_t> stop_token_ids;
    std::string lora_name;
    int num_logprobs = -1;
    int priority = 0;
    bool disable_spec_decode = false;
    bool cache_lookup = true;
    int cache_commit = 1;                       // 0 nothing, 1 the prompt's full pages, 2 prompt and generated tokens
    double timeout_s = 1e9;                     // wall-clock limit for the whole batch; overdue requests are cancelled
};

struct LLMGenerationResponse {
    std::vector<std::vector<int32_t>> output_ids;
    std::vector<std::string> output_texts;
    std::vector<FinishReason> finish_reasons;
    std::vector<std::string> errors;            // per request; empty when it succeeded
    std::vector<RequestStats> stats;
    std::vector<TokenLogprobs> logprobs;
};

// (request index, new token ids, new text — complete UTF-8 only, finished)
using StreamCallback = std::function<void(int, const std::vector<int32_t>&, const std::string&, bool)>;

class LLMInferenceRuntime {
  public:
    LLMInferenceRuntime(RuntimeOptions options, SessionFactory factory, std::shared_ptr<const Tokenizer> tokenizer,
                        std::shared_ptr<const ChatTemplate> chat_template = nullptr);
    ~LLMInferenceRuntime();
    LLMInferenceRuntime(const LLMInferenceRuntime&) = delete;

    // False when the request as a whole is malformed or the engine is unavailable (`error` says why); individual requests
    // that fail are reported in response.errors / finish_reasons and do not make the call fail.
    bool handle_request(const LLMGenerationRequest& request, LLMGenerationResponse& response, const StreamCallback& on_tokens = nullptr,
                        std::string* error = nullptr);
    std::vector<int32_t> build_prompt_ids(const LLMGenerationRequest& request, const LLMGenerationRequest::Entry& entry) const;
    int count_prompt_tokens(const LLMGenerationRequest& request, const LLMGenerationRequest::Entry& entry) const {
        return static_cast<int>(build_prompt_ids(request, entry).size());
    }

    bool capture_decoding_cuda_graph();
    std::string unavailable_reason() const;
    bool has_draft_model() const { return options_.has_draft_model; }
    bool supports_seated_admission() const { return true; }
    bool supports_stepped_execution() const { return static_cast<bool>(factory_); }
    std::shared_ptr<RequestHandle> submit(const GenerationRequest& request, std::string* why = nullptr) { return engine_->submit(request, why); }
    std::shared_ptr<RuntimeSession> open_session() const { return factory_ ? factory_() : nullptr; }
    EngineMetrics metrics() const { return engine_->metrics(); }
    RequestEngine& engine() { return *engine_; }
    void shutdown() { engine_->shutdown(); }

  private:
    RuntimeOptions options_;
    SessionFactory factory_;
    std::shared_ptr<const Tokenizer> tokenizer_;
    std::shared_ptr<const ChatTemplate> template_;
    std::unique_ptr<RequestEngine> engine_;
};

}  // namespace telb
