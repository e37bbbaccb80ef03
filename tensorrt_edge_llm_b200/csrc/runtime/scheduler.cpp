#include "scheduler.h"

#include <algorithm>

namespace telb {

static int round_up(int v, int p) { return (v + p - 1) / p * p; }
static int round_down(int v, int p) { return v / p * p; }

std::string validate_scheduling_options(const SchedulingOptions& o, const SessionCapabilities& caps) {
    if (o.max_num_tokens < 0 || o.max_chunk_tokens < 0) return "token budgets must be non-negative";
    if (o.max_num_tokens > 0 && o.max_num_tokens < caps.max_batch_size)
        return "max_num_tokens must cover one decode token per seat";
    if (o.max_chunk_tokens > 0 && o.max_chunk_tokens % caps.kv_page_size)
        return "max_chunk_tokens must be a multiple of the KV page size";
    if (o.max_num_tokens > 0 && o.max_chunk_tokens > o.max_num_tokens) return "max_chunk_tokens exceeds max_num_tokens";
    if (o.priority_reserved_slots < 0 || o.priority_reserved_slots >= std::max(caps.max_batch_size, 1))
        if (o.priority_reserved_slots != 0) return "priority_reserved_slots must leave at least one ordinary seat";
    if (o.preemption == PreemptionMode::kPause && o.max_pause_steps < 1) return "max_pause_steps must be positive with pause preemption";
    if (o.mode == IfbSchedulingMode::kMixed && !caps.compact) return "mixed scheduling needs a session that supports compact steps";
    return "";
}

ResolvedSchedulingPolicy resolve_scheduling_policy(const SchedulingOptions& o, const SessionCapabilities& caps) {
    ResolvedSchedulingPolicy r;
    const int p = std::max(caps.kv_page_size, 1);
    const int b = std::max(caps.max_batch_size, 1);
    r.mode = o.mode;
    if (r.mode == IfbSchedulingMode::kAuto) r.mode = caps.compact ? IfbSchedulingMode::kMixed : IfbSchedulingMode::kSingleCohort;
    r.policy = o.policy;
    r.preemption = o.preemption;
    const int t_max = std::max(round_down(caps.max_input_length, p), p);
    r.max_num_tokens = o.max_num_tokens > 0 ? o.max_num_tokens : std::min(round_up(512 + b, p), std::max(t_max, round_up(b + p, p)));
    r.max_chunk_tokens = o.max_chunk_tokens > 0 ? o.max_chunk_tokens : std::max(std::min(512, round_down(r.max_num_tokens - b, p)), p);
    r.priority_reserved_slots = o.priority_reserved_slots;
    r.max_pause_steps = o.max_pause_steps;
    return r;
}

StepPlan StepPlanner::plan(const std::vector<ResidentState>& residents) const {
    StepPlan plan;
    if (residents.empty()) return plan;
    std::vector<const ResidentState*> order;
    order.reserve(residents.size());
    for (const auto& r : residents) order.push_back(&r);
    std::stable_sort(order.begin(), order.end(), [&](const ResidentState* a, const ResidentState* b) {
        if (pol_.policy == SchedulingPolicy::kPriority && a->priority != b->priority) return a->priority > b->priority;
        return a->arrival < b->arrival;
    });
    // an exclusive request runs alone, as soon as it is first in line
    if (order.front()->exclusive) {
        const ResidentState* r = order.front();
        PlannedSequence s;
        s.slot = r->slot;
        s.epoch = r->epoch;
        if (r->prefilled < r->prompt_len) {
            s.kind = WorkKind::kContext;
            s.start = r->prefilled;
            s.length = std::min(r->prompt_len - r->prefilled, pol_.max_num_tokens);
            if (s.length < r->prompt_len - r->prefilled) s.length = std::max(round_down(s.length, lim_.kv_page_size), lim_.kv_page_size);
            s.last_chunk = s.start + s.length == r->prompt_len;
            plan.num_context = 1;
        } else {
            s.kind = WorkKind::kDecode;
            s.start = r->prompt_len + r->generated - 1;
            plan.num_decode = 1;
        }
        plan.total_tokens = s.length;
        plan.seqs.push_back(s);
        for (size_t i = 1; i < order.size(); ++i) plan.paused.push_back(order[i]->slot);
        return plan;
    }
    std::vector<const ResidentState*> want_ctx, want_dec;
    for (const ResidentState* r : order) {
        if (r->exclusive) { plan.paused.push_back(r->slot); continue; }
        (r->prefilled < r->prompt_len ? want_ctx : want_dec).push_back(r);
    }
    std::vector<PlannedSequence> ctx, dec;
    int budget = pol_.max_num_tokens;
    auto add_decode_rows = [&](int reserve_for_ctx) {
        for (const ResidentState* r : want_dec) {
            const bool must_run = r->paused_steps >= pol_.max_pause_steps;
            if (budget - reserve_for_ctx < 1 && !(must_run && budget >= 1)) {
                plan.paused.push_back(r->slot);
                continue;
            }
            PlannedSequence s;
            s.slot = r->slot;
            s.epoch = r->epoch;
            s.kind = WorkKind::kDecode;
            s.start = r->prompt_len + r->generated - 1;
            s.length = 1;
            dec.push_back(s);
            budget -= 1;
        }
    };
    auto add_context_chunks = [&](bool chunked) {
        for (const ResidentState* r : want_ctx) {
            const int rem = r->prompt_len - r->prefilled;
            int take = std::min(rem, budget);
            if (chunked) take = std::min(take, pol_.max_chunk_tokens);
            if (take < rem) take = round_down(take, lim_.kv_page_size);      // non-final chunks end on a page boundary
            if (take <= 0) continue;
            PlannedSequence s;
            s.slot = r->slot;
            s.epoch = r->epoch;
            s.kind = WorkKind::kContext;
            s.start = r->prefilled;
            s.length = take;
            s.last_chunk = take == rem;
            ctx.push_back(s);
            budget -= take;
        }
    };
    switch (pol_.mode) {
        case IfbSchedulingMode::kSingleCohort:
            if (!want_ctx.empty()) {
                add_context_chunks(false);
                for (const ResidentState* r : want_dec) plan.paused.push_back(r->slot);
            } else {
                add_decode_rows(0);
            }
            break;
        case IfbSchedulingMode::kPrefillFirst:
            if (!want_ctx.empty()) {
                add_context_chunks(true);
                if (ctx.empty()) add_decode_rows(0);
                else for (const ResidentState* r : want_dec) plan.paused.push_back(r->slot);
            } else {
                add_decode_rows(0);
            }
            break;
        default: {   // mixed: every decode row first (one token each), then chunked prefill in what is left
            int reserve = 0;
            if (pol_.preemption == PreemptionMode::kPause && !want_ctx.empty())
                reserve = std::min(lim_.kv_page_size, pol_.max_num_tokens - 1);   // keep room for one page of prefill
            add_decode_rows(reserve);
            add_context_chunks(true);
            break;
        }
    }
    plan.seqs = ctx;
    plan.seqs.insert(plan.seqs.end(), dec.begin(), dec.end());
    plan.num_context = static_cast<int>(ctx.size());
    plan.num_decode = static_cast<int>(dec.size());
    for (const auto& s : plan.seqs) plan.total_tokens += s.length;
    return plan;
}

// ---- request handle ---------------------------------------------------------------------------
bool RequestHandle::ready() const {
    std::lock_guard<std::mutex> lk(mu_);
    return done_;
}
std::vector<int32_t> RequestHandle::get(double timeout_s) {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait_for(lk, std::chrono::duration<double>(timeout_s), [&] { return done_; });
    if (!done_) throw std::runtime_error("request timed out");
    return tokens_;
}
TokenLogprobs RequestHandle::logprobs() const {
    std::lock_guard<std::mutex> lk(mu_);
    return logprobs_;
}
FinishReason RequestHandle::reason() const {
    std::lock_guard<std::mutex> lk(mu_);
    return reason_;
}
std::string RequestHandle::error() const {
    std::lock_guard<std::mutex> lk(mu_);
    return error_;
}
RequestStats RequestHandle::stats() const {
    std::lock_guard<std::mutex> lk(mu_);
    return stats_;
}

// ---- engine -----------------------------------------------------------------------------------
RequestEngine::RequestEngine(EngineConfig cfg, SessionFactory factory) : cfg_(cfg), factory_(std::move(factory)) {
    if (!open_session()) throw std::runtime_error("request engine: " + status_.unavailable_reason);
    thread_ = std::thread([this] { actor_loop(); });
}

RequestEngine::~RequestEngine() { shutdown(); }

bool RequestEngine::open_session() {
    try {
        session_ = factory_();
        if (!session_) throw std::runtime_error("session factory returned null");
        caps_ = session_->capabilities();
        caps_.max_batch_size = std::min(caps_.max_batch_size, std::max(cfg_.max_batch_size, 1));
        const std::string bad = validate_scheduling_options(cfg_.scheduling, caps_);
        if (!bad.empty()) throw std::runtime_error("invalid scheduling options: " + bad);
        policy_ = resolve_scheduling_policy(cfg_.scheduling, caps_);
        planner_.reset(new StepPlanner(StepPlannerLimits{caps_.max_batch_size, caps_.max_input_length, caps_.kv_page_size}, policy_));
        return true;
    } catch (const std::exception& e) {
        std::lock_guard<std::mutex> lk(mu_);
        status_.available = false;
        status_.unavailable_reason = std::string("engine_unavailable: ") + e.what();
        session_.reset();
        return false;
    }
}

std::shared_ptr<RequestHandle> RequestEngine::submit(const GenerationRequest& req, std::string* why) {
    auto refuse = [&](const char* reason) {
        if (why) *why = reason;
        ++metrics_.refused;
        return std::shared_ptr<RequestHandle>();
    };
    std::lock_guard<std::mutex> lk(mu_);
    if (stop_) return refuse("engine is shut down");
    if (!status_.available) return refuse(status_.unavailable_reason.c_str());
    if (req.priority < cfg_.scheduling.min_request_priority) return refuse("priority below the configured minimum");
    if (req.prompt_ids.empty()) return refuse("empty prompt");
    if (static_cast<int>(queue_.size()) >= cfg_.max_pending_requests) return refuse("queue_full");
    auto h = std::make_shared<RequestHandle>();
    h->id_ = next_id_++;
    h->channel_ = StreamChannel::create(true);
    h->channel_->set_stream_interval(req.stream_interval);
    h->t_submit_ = std::chrono::steady_clock::now();
    h->stats_.prompt_tokens = static_cast<int>(req.prompt_ids.size());
    queue_.push_back(Pending{h, req});
    ++metrics_.submitted;
    cv_.notify_all();
    return h;
}

void RequestEngine::cancel(uint64_t request_id) {
    std::lock_guard<std::mutex> lk(mu_);
    cancel_ids_.push_back(request_id);
    cv_.notify_all();
}

void RequestEngine::shutdown() {
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (stop_) return;
        stop_ = true;
        cv_.notify_all();
    }
    if (thread_.joinable()) thread_.join();
}

int RequestEngine::queued() const {
    std::lock_guard<std::mutex> lk(mu_);
    return static_cast<int>(queue_.size());
}
int RequestEngine::resident() const { return resident_count_.load(); }
EngineMetrics RequestEngine::metrics() const {
    std::lock_guard<std::mutex> lk(mu_);
    return metrics_;
}
EngineStatus RequestEngine::status() const {
    std::lock_guard<std::mutex> lk(mu_);
    EngineStatus s = status_;
    s.queued = static_cast<int>(queue_.size());
    s.resident = resident_count_.load();
    return s;
}
ResolvedSchedulingPolicy RequestEngine::resolved_policy() const { return policy_; }

void RequestEngine::complete_handle(const std::shared_ptr<RequestHandle>& h, FinishReason reason, const std::string& error) {
    const auto now = std::chrono::steady_clock::now();
    {
        std::lock_guard<std::mutex> lk(h->mu_);
        if (h->done_) return;
        h->done_ = true;
        h->reason_ = reason;
        h->error_ = error;
        h->stats_.generated_tokens = static_cast<int>(h->tokens_.size());
        h->stats_.total_s = std::chrono::duration<double>(now - h->t_submit_).count();
    }
    h->channel_->finish(reason);
    h->cv_.notify_all();
}

void RequestEngine::finish(Resident& r, FinishReason reason, const std::string& error) {
    try {
        if (session_) session_->release(r.st.slot);
    } catch (...) {
    }
    complete_handle(r.handle, reason, error);
    std::lock_guard<std::mutex> lk(mu_);
    if (reason == FinishReason::kCancelled) ++metrics_.cancelled;
    else if (reason == FinishReason::kError) ++metrics_.failed;
    else {
        ++metrics_.completed;
        consecutive_failures_ = 0;        // a request ran to completion: the session is healthy
    }
}

bool RequestEngine::try_admit_head() {
    Pending head;
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (queue_.empty()) return false;
        if (static_cast<int>(residents_.size()) >= caps_.max_batch_size) { ++metrics_.stalls_no_capacity; return false; }
        // seats held back for high-priority requests
        const int free_seats = caps_.max_batch_size - static_cast<int>(residents_.size());
        if (queue_.front().req.priority <= cfg_.scheduling.min_request_priority && free_seats <= policy_.priority_reserved_slots &&
            policy_.priority_reserved_slots > 0) {
            ++metrics_.stalls_no_capacity;
            return false;
        }
        // an exclusive resident, or an exclusive head behind residents, blocks admission
        for (const auto& kv : residents_)
            if (kv.second.st.exclusive) { ++metrics_.stalls_exclusive; return false; }
        if (queue_.front().req.exclusive && !residents_.empty()) { ++metrics_.stalls_exclusive; return false; }
        head = queue_.front();
        queue_.pop_front();
    }
    if (head.handle->channel_->cancelled()) {
        complete_handle(head.handle, FinishReason::kCancelled, "");
        std::lock_guard<std::mutex> lk(mu_);
        ++metrics_.cancelled;
        return true;
    }
    AdmissionResult ar;
    try {
        ar = session_->admit(head.handle->id_, head.req);
    } catch (const std::exception& e) {
        ar.admitted = false;
        ar.retry_later = false;
        ar.reason = e.what();
    }
    if (!ar.admitted) {
        if (ar.retry_later && !residents_.empty()) {     // capacity will free up: put it back at the head
            std::lock_guard<std::mutex> lk(mu_);
            queue_.push_front(head);
            ++metrics_.stalls_no_capacity;
            return false;
        }
        complete_handle(head.handle, FinishReason::kError, ar.reason.empty() ? "admission refused" : ar.reason);
        std::lock_guard<std::mutex> lk(mu_);
        ++metrics_.failed;
        return true;
    }
    Resident r;
    r.handle = head.handle;
    r.req = head.req;
    r.st.slot = ar.slot;
    r.st.prompt_len = static_cast<int>(head.req.prompt_ids.size());
    r.st.prefilled = ar.reused_tokens;
    r.st.priority = head.req.priority;
    r.st.exclusive = head.req.exclusive;
    r.st.arrival = arrival_++;
    const auto now = std::chrono::steady_clock::now();
    {
        std::lock_guard<std::mutex> hl(head.handle->mu_);
        head.handle->t_admit_ = now;
        head.handle->stats_.queue_s = std::chrono::duration<double>(now - head.handle->t_submit_).count();
        head.handle->stats_.reused_tokens = ar.reused_tokens;
    }
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (!residents_.empty()) ++metrics_.admitted_mid_flight;
        metrics_.queue_latency_s_sum += head.handle->stats_.queue_s;
        metrics_.prefix_reused_tokens += ar.reused_tokens;
    }
    residents_[ar.slot] = std::move(r);
    resident_count_.store(static_cast<int>(residents_.size()));
    return true;
}

void RequestEngine::fail_session(const std::string& why) {
    for (auto& kv : residents_) complete_handle(kv.second.handle, FinishReason::kError, why);
    {
        std::lock_guard<std::mutex> lk(mu_);
        metrics_.failed += residents_.size();
        ++metrics_.session_failures;
    }
    residents_.clear();
    resident_count_.store(0);
    session_.reset();
    ++consecutive_failures_;
    if (consecutive_failures_ >= cfg_.max_consecutive_session_failures || !open_session()) {
        std::deque<Pending> drop;
        {
            std::lock_guard<std::mutex> lk(mu_);
            status_.available = false;
            if (status_.unavailable_reason.empty()) status_.unavailable_reason = "engine_unavailable: " + why;
            drop.swap(queue_);
            metrics_.failed += drop.size();
        }
        for (auto& p : drop) complete_handle(p.handle, FinishReason::kError, "engine_unavailable");
    }
}

void RequestEngine::run_step() {
    std::vector<ResidentState> states;
    states.reserve(residents_.size());
    for (auto& kv : residents_) states.push_back(kv.second.st);
    const StepPlan plan = planner_->plan(states);
    for (int slot : plan.paused) {
        auto it = residents_.find(slot);
        if (it != residents_.end()) ++it->second.st.paused_steps;
    }
    if (plan.empty()) return;
    StepResult res;
    try {
        res = session_->execute(plan);
    } catch (const std::exception& e) {
        fail_session(e.what());
        return;
    }
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (plan.num_context && plan.num_decode) ++metrics_.mixed_steps;
        else if (plan.num_context) ++metrics_.prompt_steps;
        else ++metrics_.decode_steps;
        metrics_.step_tokens += plan.total_tokens;
        metrics_.paused_resident_steps += plan.paused.size();
    }
    for (const auto& s : plan.seqs) {
        auto it = residents_.find(s.slot);
        if (it == residents_.end()) continue;
        it->second.st.paused_steps = 0;
        if (s.kind == WorkKind::kContext) it->second.st.prefilled += s.length;
    }
    for (const auto& d : res.deltas) {
        auto it = residents_.find(d.slot);
        if (it == residents_.end()) continue;
        Resident& r = it->second;
        if (!d.tokens.empty()) {
            {
                std::lock_guard<std::mutex> hl(r.handle->mu_);
                if (r.handle->tokens_.empty()) {
                    r.handle->t_first_ = std::chrono::steady_clock::now();
                    r.handle->stats_.ttft_s = std::chrono::duration<double>(r.handle->t_first_ - r.handle->t_submit_).count();
                }
                r.handle->tokens_.insert(r.handle->tokens_.end(), d.tokens.begin(), d.tokens.end());
                r.handle->logprobs_.append(d.logprobs);
            }
            r.st.generated += static_cast<int>(d.tokens.size());
            r.handle->channel_->push(d.tokens, d.logprobs);
        }
        FinishReason why = d.finished ? d.reason : FinishReason::kNotFinished;
        if (why == FinishReason::kNotFinished && r.st.generated >= r.req.max_tokens) why = FinishReason::kLength;
        if (why != FinishReason::kNotFinished) {
            finish(r, why);
            residents_.erase(it);
        }
    }
    resident_count_.store(static_cast<int>(residents_.size()));
}

void RequestEngine::actor_loop() {
    for (;;) {
        std::vector<uint64_t> cancels;
        {
            std::unique_lock<std::mutex> lk(mu_);
            if (stop_) break;
            if (queue_.empty() && residents_.empty() && cancel_ids_.empty())
                cv_.wait_for(lk, std::chrono::duration<double>(cfg_.idle_wait_s));
            if (stop_) break;
            cancels.swap(cancel_ids_);
        }
        if (!session_) {
            std::this_thread::sleep_for(std::chrono::duration<double>(cfg_.idle_wait_s));
            continue;
        }
        // cancellations (explicit ids and consumers that went away)
        for (auto it = residents_.begin(); it != residents_.end();) {
            const bool hit = it->second.handle->channel_->cancelled() ||
                             std::find(cancels.begin(), cancels.end(), it->second.handle->id_) != cancels.end();
            if (hit) {
                finish(it->second, FinishReason::kCancelled);
                it = residents_.erase(it);
            } else {
                ++it;
            }
        }
        if (!cancels.empty()) {
            std::lock_guard<std::mutex> lk(mu_);
            for (auto& p : queue_)
                if (std::find(cancels.begin(), cancels.end(), p.handle->id_) != cancels.end()) p.handle->channel_->cancel();
        }
        resident_count_.store(static_cast<int>(residents_.size()));
        while (session_ && try_admit_head()) {
        }
        if (session_ && !residents_.empty()) run_step();
    }
    // shutdown: everything still in flight is cancelled
    for (auto& kv : residents_) finish(kv.second, FinishReason::kCancelled);
    residents_.clear();
    resident_count_.store(0);
    std::deque<Pending> drop;
    {
        std::lock_guard<std::mutex> lk(mu_);
        drop.swap(queue_);
    }
    for (auto& p : drop) complete_handle(p.handle, FinishReason::kCancelled, "");
}

}  // namespace telb
