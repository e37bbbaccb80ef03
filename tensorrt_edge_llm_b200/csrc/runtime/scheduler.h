// In-flight batching: scheduling options, the step planner and the request-engine actor.
//
// Counterparts in the reference: cpp/scheduler/schedulingPolicy.h:34-108 (modes, policy,
// preemption, defaults), cpp/scheduler/stepPlanner.h:34-150 (ResidentState, StepPlan, planning
// rules), cpp/scheduler/requestEngine.{h,cpp} (actor loop, admission, failure scopes, metrics) and
// the session seam cpp/runtime/runtimeSession.h:162-291.  The design note is
// docs/source/developer_guide/software-design/in-flight-batching.md.
//
// The engine owns ONE thread.  All mutable scheduler state lives on that thread; callers talk to
// it through a bounded command queue and read results from per-request stream channels.  The
// model is reached through the abstract RuntimeSession, so the scheduler is testable with a
// scripted session and no GPU.
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "streaming.h"

namespace telb {

// ---- policy ------------------------------------------------------------------------------------
enum class IfbSchedulingMode { kAuto = 0, kMixed, kPrefillFirst, kSingleCohort };
enum class SchedulingPolicy { kFcfs = 0, kPriority };
enum class PreemptionMode { kNone = 0, kPause };

struct SchedulingOptions {
    IfbSchedulingMode mode = IfbSchedulingMode::kAuto;
    SchedulingPolicy policy = SchedulingPolicy::kFcfs;
    PreemptionMode preemption = PreemptionMode::kNone;
    int max_num_tokens = 0;            // 0 = derive from the session's limits
    int max_chunk_tokens = 0;          // 0 = derive
    int priority_reserved_slots = 0;   // seats kept free for requests above min priority
    int max_pause_steps = 8;           // a paused decode row is resumed after this many steps
    int min_request_priority = 0;      // requests below are refused (HTTP 400 at the server)
};

struct SessionCapabilities {
    bool compact = true;               // prefill chunks and decode rows may share one step
    int max_batch_size = 1;
    int max_input_length = 2048;
    int kv_page_size = 64;
    int max_kv_tokens = 4096;          // per sequence
};

struct ResolvedSchedulingPolicy {
    IfbSchedulingMode mode = IfbSchedulingMode::kMixed;
    SchedulingPolicy policy = SchedulingPolicy::kFcfs;
    PreemptionMode preemption = PreemptionMode::kNone;
    int max_num_tokens = 0;
    int max_chunk_tokens = 0;
    int priority_reserved_slots = 0;
    int max_pause_steps = 8;
};

// Empty string when valid, else a human-readable reason.
std::string validate_scheduling_options(const SchedulingOptions& o, const SessionCapabilities& caps);
ResolvedSchedulingPolicy resolve_scheduling_policy(const SchedulingOptions& o, const SessionCapabilities& caps);

// ---- planner -----------------------------------------------------------------------------------
struct ResidentState {
    int slot = -1;
    uint32_t epoch = 0;
    int prompt_len = 0;
    int prefilled = 0;        // prompt tokens already in the KV cache
    int generated = 0;
    int priority = 0;
    uint64_t arrival = 0;     // admission order
    int paused_steps = 0;     // consecutive steps this row has been paused
    bool exclusive = false;   // must run alone (e.g. guided decoding)
};

struct StepPlannerLimits {
    int max_batch_size = 1;
    int max_input_length = 2048;
    int kv_page_size = 64;
};

enum class WorkKind { kContext = 0, kDecode = 1 };

struct PlannedSequence {
    int slot = -1;
    uint32_t epoch = 0;
    WorkKind kind = WorkKind::kDecode;
    int start = 0;            // first prompt token of the chunk (context) or position of the fed token (decode)
    int length = 1;           // tokens executed this step
    bool last_chunk = false;  // context: this chunk completes the prompt, so the step samples a token
};

struct StepPlan {
    std::vector<PlannedSequence> seqs;     // context chunks first, then decode rows (compact layout)
    std::vector<int> paused;               // slots skipped this step
    int num_context = 0, num_decode = 0, total_tokens = 0;
    bool empty() const { return seqs.empty(); }
};

class StepPlanner {
  public:
    StepPlanner(StepPlannerLimits limits, ResolvedSchedulingPolicy policy) : lim_(limits), pol_(policy) {}
    StepPlan plan(const std::vector<ResidentState>& residents) const;
    const ResolvedSchedulingPolicy& policy() const { return pol_; }

  private:
    StepPlannerLimits lim_;
    ResolvedSchedulingPolicy pol_;
};

// ---- session seam ------------------------------------------------------------------------------
struct GenerationRequest {
    std::vector<int32_t> prompt_ids;
    int max_tokens = 128;
    float temperature = 0.f;
    int top_k = 0;
    float top_p = 1.f;
    uint64_t seed = 42;
    bool ignore_eos = false;
    std::vector<int32_t> stop_token_ids;
    int priority = 0;
    bool exclusive = false;
    std::string lora_name;
    int stream_interval = 1;
    int num_logprobs = -1;                  // -1 = none; 0 = the chosen token's only; k = plus the k most likely
    std::string guided_type;                // "", "json_object", "json_schema", "regex", "choice"
    std::string guided_spec;                // JSON text of the constraint's parameters
    std::vector<int32_t> logit_bias_ids;    // additive bias on these token ids ...
    std::vector<float> logit_bias_values;   // ... by these amounts, before sampling
    // Context (prefix) cache policies of this request: look the prompt up at admission or bypass the cache; publish
    // nothing (0), the prompt's full pages (1, "prefill_state_only") or prompt plus generated tokens (2).
    bool cache_lookup = true;
    int cache_commit = 1;
    bool disable_spec_decode = false;       // decode this request token by token even on a speculative deployment
    int64_t embeds_key = 0;                 // non-zero: the session holds prompt embedding rows (multimodal prompt) under this key
};

struct AdmissionResult {
    bool admitted = false;
    int slot = -1;
    int reused_tokens = 0;        // prompt tokens served from the prefix cache
    std::string reason;           // why not, when refused
    bool retry_later = true;      // false = permanent (prompt too long ...)
};

struct TokenDelta {
    int slot = -1;
    std::vector<int32_t> tokens;
    TokenLogprobs logprobs;                 // empty unless the request asked for them
    bool finished = false;
    FinishReason reason = FinishReason::kNotFinished;
};

struct StepResult {
    std::vector<TokenDelta> deltas;
};

class SessionLostError : public std::runtime_error {
  public:
    using std::runtime_error::runtime_error;
};

class RuntimeSession {
  public:
    virtual ~RuntimeSession() = default;
    virtual SessionCapabilities capabilities() const = 0;
    virtual AdmissionResult admit(uint64_t request_id, const GenerationRequest& req) = 0;
    virtual StepResult execute(const StepPlan& plan) = 0;     // may throw; SessionLostError = session unusable
    virtual void release(int slot) = 0;                       // request left (finished / cancelled / failed)
};
using SessionFactory = std::function<std::shared_ptr<RuntimeSession>()>;

// ---- engine ------------------------------------------------------------------------------------
struct EngineConfig {
    int command_queue_capacity = 64;
    int max_pending_requests = 256;
    int max_batch_size = 1;
    int max_consecutive_session_failures = 2;
    double idle_wait_s = 0.05;
    SchedulingOptions scheduling;
};

struct EngineMetrics {
    uint64_t submitted = 0, refused = 0, completed = 0, cancelled = 0, failed = 0;
    uint64_t admitted_mid_flight = 0;
    uint64_t stalls_no_capacity = 0, stalls_exclusive = 0;
    uint64_t decode_steps = 0, prompt_steps = 0, mixed_steps = 0, step_tokens = 0;
    uint64_t paused_resident_steps = 0, session_failures = 0, prefix_reused_tokens = 0;
    double queue_latency_s_sum = 0.0;
};

struct EngineStatus {
    bool available = true;
    std::string unavailable_reason;
    int queued = 0, resident = 0;
};

struct RequestStats {
    int prompt_tokens = 0, generated_tokens = 0, reused_tokens = 0;
    double queue_s = 0.0, ttft_s = 0.0, total_s = 0.0;
};

class RequestHandle {
  public:
    uint64_t id() const { return id_; }
    std::shared_ptr<StreamChannel> stream() const { return channel_; }
    bool ready() const;
    // Blocks until the request finishes; returns all generated tokens.
    std::vector<int32_t> get(double timeout_s = 1e9);
    TokenLogprobs logprobs() const;         // of the tokens generated so far
    FinishReason reason() const;
    std::string error() const;
    void cancel() { channel_->cancel(); }
    RequestStats stats() const;

  private:
    friend class RequestEngine;
    uint64_t id_ = 0;
    std::shared_ptr<StreamChannel> channel_;
    mutable std::mutex mu_;
    std::condition_variable cv_;
    bool done_ = false;
    std::vector<int32_t> tokens_;
    TokenLogprobs logprobs_;
    FinishReason reason_ = FinishReason::kNotFinished;
    std::string error_;
    RequestStats stats_;
    std::chrono::steady_clock::time_point t_submit_, t_admit_, t_first_;
};

class RequestEngine {
  public:
    RequestEngine(EngineConfig cfg, SessionFactory factory);
    ~RequestEngine();
    RequestEngine(const RequestEngine&) = delete;

    // Returns null (and bumps `refused`) when the queue is full, the priority is below the floor or
    // the engine is unavailable; `why` receives the reason.
    std::shared_ptr<RequestHandle> submit(const GenerationRequest& req, std::string* why = nullptr);
    void cancel(uint64_t request_id);
    void shutdown();
    int queued() const;
    int resident() const;
    EngineMetrics metrics() const;
    EngineStatus status() const;
    ResolvedSchedulingPolicy resolved_policy() const;

  private:
    struct Pending {
        std::shared_ptr<RequestHandle> handle;
        GenerationRequest req;
    };
    struct Resident {
        std::shared_ptr<RequestHandle> handle;
        GenerationRequest req;
        ResidentState st;
    };
    void actor_loop();
    bool open_session();
    bool try_admit_head();
    void run_step();
    void finish(Resident& r, FinishReason reason, const std::string& error = "");
    void fail_session(const std::string& why);
    void complete_handle(const std::shared_ptr<RequestHandle>& h, FinishReason reason, const std::string& error);

    EngineConfig cfg_;
    SessionFactory factory_;
    std::shared_ptr<RuntimeSession> session_;
    SessionCapabilities caps_;
    ResolvedSchedulingPolicy policy_;
    std::unique_ptr<StepPlanner> planner_;

    mutable std::mutex mu_;                 // guards queue_, cancel_ids_, metrics_, status_, counters below
    std::condition_variable cv_;
    std::deque<Pending> queue_;
    std::vector<uint64_t> cancel_ids_;
    EngineMetrics metrics_;
    EngineStatus status_;
    bool stop_ = false;
    uint64_t next_id_ = 1, arrival_ = 0;
    int consecutive_failures_ = 0;
    std::atomic<int> resident_count_{0};

    std::map<int, Resident> residents_;     // actor-thread only, keyed by slot
    std::thread thread_;
};

}  // namespace telb
