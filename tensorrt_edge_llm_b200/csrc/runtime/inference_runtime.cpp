#include "inference_runtime.h"

#include <algorithm>
#include <chrono>

#include "streaming.h"

namespace telb {

LLMInferenceRuntime::LLMInferenceRuntime(RuntimeOptions options, SessionFactory factory, std::shared_ptr<const Tokenizer> tokenizer,
                                         std::shared_ptr<const ChatTemplate> chat_template)
    : options_(std::move(options)), factory_(std::move(factory)), tokenizer_(std::move(tokenizer)), template_(std::move(chat_template)) {
    if (!factory_) throw std::invalid_argument("LLMInferenceRuntime needs a session factory");
    if (!tokenizer_) throw std::invalid_argument("LLMInferenceRuntime needs a tokenizer");
    engine_ = std::make_unique<RequestEngine>(options_.engine, factory_);
}

LLMInferenceRuntime::~LLMInferenceRuntime() { engine_->shutdown(); }

std::vector<int32_t> LLMInferenceRuntime::build_prompt_ids(const LLMGenerationRequest& request,
                                                           const LLMGenerationRequest::Entry& entry) const {
    if (!entry.prompt_ids.empty()) return entry.prompt_ids;
    if (!entry.messages.empty()) {
        if (request.apply_chat_template && template_)
            return tokenizer_->encode(template_->apply(entry.messages, request.add_generation_prompt, request.enable_thinking), false);
        std::string text;                        // no template: the contents, one per line
        for (const auto& m : entry.messages) {
            if (!text.empty()) text += "\n";
            text += m.content;
        }
        return tokenizer_->encode(text, true);
    }
    return tokenizer_->encode(entry.prompt, true);
}

bool LLMInferenceRuntime::capture_decoding_cuda_graph() {
    if (!options_.capture_hook) return true;
    if (engine_->queued() > 0 || engine_->resident() > 0) return false;      // never beside a running step
    return options_.capture_hook();
}

std::string LLMInferenceRuntime::unavailable_reason() const {
    const EngineStatus s = engine_->status();
    return s.available ? std::string() : s.unavailable_reason;
}

namespace {

struct Live {
    std::shared_ptr<RequestHandle> handle;
    std::string pending_bytes;       // bytes of tokens whose UTF-8 sequence is not complete yet
    size_t scanned = 0;              // text before this offset holds no stop sequence (minus the longest stop's overlap)
    bool done = false;
    bool stopped = false;            // a textual stop sequence ended it
};

}  // namespace

bool LLMInferenceRuntime::handle_request(const LLMGenerationRequest& request, LLMGenerationResponse& response,
                                         const StreamCallback& on_tokens, std::string* error) {
    auto fail = [&](const std::string& why) {
        if (error) *error = why;
        return false;
    };
    const int n = static_cast<int>(request.requests.size());
    if (n == 0) return fail("empty request batch");
    if (request.max_generate_length < 1) return fail("max_generate_length must be positive");
    for (const auto& s : request.stop)
        if (s.empty()) return fail("empty stop sequence");
    const std::string unavailable = unavailable_reason();
    if (!unavailable.empty()) return fail("runtime unavailable: " + unavailable);

    response = LLMGenerationResponse();
    response.output_ids.resize(n);
    response.output_texts.resize(n);
    response.finish_reasons.assign(n, FinishReason::kNotFinished);
    response.errors.resize(n);
    response.stats.resize(n);
    response.logprobs.resize(n);

    size_t max_stop = 0;
    for (const auto& s : request.stop) max_stop = std::max(max_stop, s.size());

    std::vector<Live> live(n);
    int open = 0;
    for (int i = 0; i < n; ++i) {
        GenerationRequest g;
        g.prompt_ids = build_prompt_ids(request, request.requests[i]);
        if (g.prompt_ids.empty()) {
            response.errors[i] = "empty prompt";
            response.finish_reasons[i] = FinishReason::kError;
            live[i].done = true;
            continue;
        }
        g.max_tokens = request.max_generate_length;
        g.temperature = request.temperature;
        g.top_k = request.top_k;
        g.top_p = request.top_p;
        g.seed = request.seed + static_cast<uint64_t>(i);
        g.ignore_eos = request.ignore_eos;
        g.stop_token_ids = request.stop_token_ids;
        g.priority = request.priority;
        g.lora_name = request.lora_name;
        g.num_logprobs = request.num_logprobs;
        g.cache_lookup = request.cache_lookup;
        g.cache_commit = request.cache_commit;
        g.disable_spec_decode = request.disable_spec_decode;
        std::string why;
        live[i].handle = engine_->submit(g, &why);
        if (!live[i].handle) {
            response.errors[i] = why.empty() ? "refused" : why;
            response.finish_reasons[i] = FinishReason::kError;
            live[i].done = true;
            continue;
        }
        ++open;
    }

    const auto t0 = std::chrono::steady_clock::now();
    auto emit = [&](int i, const std::vector<int32_t>& toks, bool finished) {
        Live& l = live[i];
        std::string fresh;
        if (!l.stopped) {
            auto& ids = response.output_ids[i];
            ids.insert(ids.end(), toks.begin(), toks.end());
            for (int32_t t : toks)
                if (!tokenizer_->is_special(t)) l.pending_bytes += tokenizer_->id_to_bytes(t);
            const size_t ok = finished ? l.pending_bytes.size() : utf8_complete_prefix(l.pending_bytes);
            fresh = l.pending_bytes.substr(0, ok);
            l.pending_bytes.erase(0, ok);
            std::string& text = response.output_texts[i];
            const size_t before = text.size();
            text += fresh;
            if (max_stop > 0) {
                const size_t from = l.scanned > max_stop ? l.scanned - max_stop : 0;
                size_t cut = std::string::npos;
                for (const auto& s : request.stop) cut = std::min(cut, text.find(s, from));
                if (cut != std::string::npos) {
                    text.erase(cut);
                    fresh = cut > before ? text.substr(before) : std::string();
                    l.stopped = true;
                    l.handle->cancel();
                } else {
                    l.scanned = text.size();
                }
            }
        }
        if (on_tokens && (!fresh.empty() || !toks.empty() || finished)) on_tokens(i, l.stopped ? std::vector<int32_t>() : toks, fresh, finished);
    };

    auto finalize = [&](int i) {
        Live& l = live[i];
        l.done = true;
        --open;
        l.handle->get(5.0);                      // the finishing chunk is pushed just before the handle's record is complete
        FinishReason r = l.handle->reason();
        if (l.stopped) r = FinishReason::kStopWords;
        response.finish_reasons[i] = r;
        response.errors[i] = l.stopped ? std::string() : l.handle->error();
        response.stats[i] = l.handle->stats();
        response.logprobs[i] = l.handle->logprobs();
    };
    while (open > 0) {
        bool any = false;
        int first_open = -1;
        for (int i = 0; i < n; ++i) {
            Live& l = live[i];
            if (l.done) continue;
            if (first_open < 0) first_open = i;
            StreamChunk chunk;
            while (!l.done && l.handle->stream()->try_pop(chunk)) {
                any = true;
                emit(i, chunk.token_ids, chunk.finished);
                if (chunk.finished) finalize(i);
            }
        }
        if (!any && open > 0 && first_open >= 0 && !live[first_open].done) {
            // nothing queued anywhere: sleep on one open channel instead of spinning
            StreamChunk chunk;
            if (live[first_open].handle->stream()->wait_pop(chunk, 0.02)) {
                emit(first_open, chunk.token_ids, chunk.finished);
                if (chunk.finished) finalize(first_open);
            }
        }
        if (open > 0 && std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > request.timeout_s) {
            for (auto& l : live)
                if (!l.done && l.handle) l.handle->cancel();
        }
    }
    return true;
}

}  // namespace telb
