// Concurrency check of the native runtime, meant to be built with a sanitizer (`python -m tensorrt_edge_llm_b200.build
// --sanitize thread` or `address`): many client threads submit, stream, poll metrics and cancel against one request
// engine whose actor thread drives a scripted session, while the streaming channels are consumed from other threads.
// A second phase drives the runtime façade the same way: several threads call handle_request on one LLMInferenceRuntime at
// once (each with a batch of its own, a streaming callback and, for some, a textual stop sequence).
// The program checks the results itself (every finished request carries exactly the tokens the scripted session emits)
// and exits non-zero on a mismatch; data races and memory errors are the sanitizer's to report.
//
// Reference counterpart: the reference has no race-detection target; its engine is exercised by unit tests only
// (tests/cpp/runtime/requestEngineTests.cpp).
#include <atomic>
#include <chrono>
#include <cstdio>
#include <map>
#include <thread>
#include <vector>

#include "../inference_runtime.h"
#include "../scheduler.h"
#include "../streaming.h"

using namespace telb;

namespace {

// Emits prompt_ids[0] + k as the k-th generated token; one token per decode row and per completed prompt.
class ScriptedSession : public RuntimeSession {
  public:
    SessionCapabilities capabilities() const override {
        SessionCapabilities c;
        c.max_batch_size = 8;
        c.max_input_length = 512;
        c.max_kv_tokens = 2048;
        return c;
    }
    AdmissionResult admit(uint64_t, const GenerationRequest& req) override {
        AdmissionResult r;
        for (int s = 0; s < 8; ++s) {
            if (!busy_[s]) {
                busy_[s] = true;
                base_[s] = req.prompt_ids.empty() ? 0 : req.prompt_ids[0];
                count_[s] = 0;
                r.admitted = true;
                r.slot = s;
                return r;
            }
        }
        r.reason = "no free seat";
        return r;
    }
    StepResult execute(const StepPlan& plan) override {
        StepResult out;
        for (const PlannedSequence& q : plan.seqs) {
            if (q.kind == WorkKind::kContext && !q.last_chunk) continue;
            TokenDelta d;
            d.slot = q.slot;
            d.tokens.push_back(base_[q.slot] + count_[q.slot]++);
            out.deltas.push_back(d);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
        return out;
    }
    void release(int slot) override { busy_[slot] = false; }

  private:
    bool busy_[8] = {false, false, false, false, false, false, false, false};
    int32_t base_[8] = {0};
    int count_[8] = {0};
};

}  // namespace

int main() {
    EngineConfig cfg;
    cfg.max_batch_size = 8;
    cfg.max_pending_requests = 512;
    cfg.command_queue_capacity = 512;
    cfg.scheduling.max_num_tokens = 256;
    RequestEngine engine(cfg, [] { return std::make_shared<ScriptedSession>(); });
    std::atomic<int> bad{0}, done{0}, cancelled{0};
    std::atomic<bool> stop{false};
    std::thread poller([&] {            // a monitoring client: metrics and status while everything else runs
        while (!stop.load()) {
            const EngineMetrics m = engine.metrics();
            const EngineStatus s = engine.status();
            if (m.completed > m.submitted || s.resident > 8) bad.fetch_add(1);
            (void)engine.queued();
            std::this_thread::sleep_for(std::chrono::microseconds(200));
        }
    });
    std::vector<std::thread> clients;
    for (int c = 0; c < 6; ++c) {
        clients.emplace_back([&, c] {
            for (int i = 0; i < 40; ++i) {
                GenerationRequest req;
                const int base = 1000 * c + 10 * i;
                req.prompt_ids.assign(3 + (i % 40), base);
                req.max_tokens = 4 + (i % 9);
                req.ignore_eos = true;
                req.priority = i % 3;
                std::string why;
                std::shared_ptr<RequestHandle> h = engine.submit(req, &why);
                if (!h) continue;                                 // refused under load: allowed
                const bool cancel_it = (i % 7) == 3;
                std::vector<int32_t> streamed;
                std::thread consumer([&] {                        // the streaming consumer of this request
                    StreamChunk ch;
                    while (h->stream()->wait_pop(ch, 5.0)) {
                        streamed.insert(streamed.end(), ch.token_ids.begin(), ch.token_ids.end());
                        if (cancel_it && streamed.size() >= 2) h->cancel();
                        if (ch.finished) break;
                    }
                });
                const std::vector<int32_t> got = h->get(30.0);
                consumer.join();
                if (cancel_it && h->reason() == FinishReason::kCancelled) {
                    cancelled.fetch_add(1);
                } else {
                    if ((int)got.size() != req.max_tokens && !cancel_it) bad.fetch_add(1);
                    for (size_t k = 0; k < got.size(); ++k)
                        if (got[k] != base + (int)k) bad.fetch_add(1);
                }
                if (streamed.size() > got.size()) bad.fetch_add(1);
                done.fetch_add(1);
                (void)h->stats();
            }
        });
    }
    for (std::thread& t : clients) t.join();
    stop.store(true);
    poller.join();
    engine.shutdown();
    const EngineMetrics m = engine.metrics();
    std::printf("requests %d cancelled %d mismatches %d engine: submitted %llu completed %llu cancelled %llu failed %llu\n", done.load(),
                cancelled.load(), bad.load(), (unsigned long long)m.submitted, (unsigned long long)m.completed,
                (unsigned long long)m.cancelled, (unsigned long long)m.failed);
    if (!(bad.load() == 0 && done.load() > 0 && m.failed == 0)) return 1;

    // ---- phase 2: concurrent handle_request calls on the façade ----
    // a byte-level vocabulary of the 26 lower-case letters: token i decodes to the letter 'a' + i
    std::string vocab;
    for (int i = 0; i < 26; ++i) {
        if (i) vocab += ",";
        vocab += std::string("\"") + static_cast<char>('a' + i) + "\":" + std::to_string(i);
    }
    const std::string tok_json = "{\"model\":{\"type\":\"BPE\",\"vocab\":{" + vocab + "},\"merges\":[]},\"added_tokens\":[]}";
    auto tokenizer = std::make_shared<Tokenizer>(Tokenizer::from_json_text(tok_json));
    RuntimeOptions opt;
    opt.engine = cfg;
    std::atomic<int> hooks{0};
    opt.capture_hook = [&] { hooks.fetch_add(1); return true; };
    LLMInferenceRuntime runtime(opt, [] { return std::make_shared<ScriptedSession>(); }, tokenizer);
    std::atomic<int> bad2{0}, batches{0}, pieces{0};
    std::vector<std::thread> callers;
    for (int c = 0; c < 5; ++c) {
        callers.emplace_back([&, c] {
            for (int i = 0; i < 12; ++i) {
                LLMGenerationRequest req;
                req.max_generate_length = 5 + (i % 4);
                req.ignore_eos = true;
                const int n = 1 + (i + c) % 3;
                for (int k = 0; k < n; ++k) {
                    LLMGenerationRequest::Entry e;
                    e.prompt_ids.assign(2 + k, (c + i + k) % 8);         // generates the letters from 'a' + base on
                    req.requests.push_back(e);
                }
                const bool with_stop = (i % 5) == 2;
                if (with_stop) req.stop = {"j"};                          // bases 0..7, up to 8 tokens: 'j' is token 9
                LLMGenerationResponse resp;
                std::string err;
                std::vector<std::string> streamed(n);
                const bool ok = runtime.handle_request(req, resp, [&](int idx, const std::vector<int32_t>&, const std::string& text, bool) {
                    streamed[idx] += text;
                    pieces.fetch_add(1);
                }, &err);
                if (!ok) {
                    bad2.fetch_add(1);
                    continue;
                }
                for (int k = 0; k < n; ++k) {
                    const int base = (c + i + k) % 8;
                    std::string want;
                    for (int t = 0; t < req.max_generate_length; ++t) want += static_cast<char>('a' + base + t);
                    if (with_stop) {
                        const size_t cut = want.find('j');
                        if (cut != std::string::npos) want.erase(cut);
                    }
                    if (resp.output_texts[k] != want || streamed[k] != want) bad2.fetch_add(1);
                    if (!resp.errors[k].empty()) bad2.fetch_add(1);
                }
                batches.fetch_add(1);
                (void)runtime.metrics();
                (void)runtime.unavailable_reason();
            }
        });
    }
    for (std::thread& t : callers) t.join();
    while (runtime.engine().resident() > 0 || runtime.engine().queued() > 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    const bool captured = runtime.capture_decoding_cuda_graph();
    runtime.shutdown();
    std::printf("facade: batches %d streamed pieces %d mismatches %d capture hook %d\n", batches.load(), pieces.load(), bad2.load(), hooks.load());
    return (bad2.load() == 0 && batches.load() == 60 && captured && hooks.load() == 1) ? 0 : 1;
}
