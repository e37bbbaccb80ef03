// Python bindings of the native runtime (module `_telb_runtime`).
//
// Counterpart of python/nanobind/bindings.cpp in the reference (LLMRuntime, StreamChannel,
// RequestHandle, RequestEngine, validate_scheduling_options ...).  The model executor is reached
// through RuntimeSession, which Python subclasses (the PyTorch model runner); every call from the
// engine's actor thread into Python takes the GIL, and blocking native calls release it.
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "inference_runtime.h"
#include "json.h"
#include "media.h"
#include "multistage.h"
#include "paged_kv.h"
#include "ple.h"
#include "runtime_core.h"
#include "scheduler.h"
#include "streaming.h"
#include "tokenizer.h"

namespace py = pybind11;
using namespace telb;

class PyRuntimeSession : public RuntimeSession {
  public:
    using RuntimeSession::RuntimeSession;
    SessionCapabilities capabilities() const override {
        PYBIND11_OVERRIDE_PURE(SessionCapabilities, RuntimeSession, capabilities, );
    }
    AdmissionResult admit(uint64_t request_id, const GenerationRequest& req) override {
        PYBIND11_OVERRIDE_PURE(AdmissionResult, RuntimeSession, admit, request_id, req);
    }
    StepResult execute(const StepPlan& plan) override { PYBIND11_OVERRIDE_PURE(StepResult, RuntimeSession, execute, plan); }
    void release(int slot) override { PYBIND11_OVERRIDE_PURE(void, RuntimeSession, release, slot); }
};

// A session factory backed by a Python callable.  The factory and the sessions it returns are Python objects: the GIL is held
// around every use, and a returned session keeps its Python object alive for as long as native code holds the pointer.
static SessionFactory session_factory_from_python(py::function factory) {
    auto shared_factory = std::make_shared<py::function>(std::move(factory));
    return [shared_factory]() {
        py::gil_scoped_acquire gil;
        py::object obj = (*shared_factory)();
        auto sp = obj.cast<std::shared_ptr<RuntimeSession>>();
        auto keep = std::make_shared<py::object>(std::move(obj));
        return std::shared_ptr<RuntimeSession>(sp.get(), [sp, keep](RuntimeSession*) mutable {
            py::gil_scoped_acquire g;
            keep.reset();
            sp.reset();
        });
    };
}

// ---- stage-graph values ↔ Python ----------------------------------------------------------------------------------------
// str and bytes travel as native text / bytes, a plain list of ints as token ids; token ids and float tensors made by
// native stages become a list / a numpy array; every other Python object rides through the graph untouched as an opaque handle.
namespace msg = telb::multistage;

static msg::PortValue port_from_python(const py::handle& h) {
    if (h.is_none()) return msg::PortValue();
    if (py::isinstance<py::str>(h)) return msg::PortValue::text(h.cast<std::string>());
    if (py::isinstance<py::bytes>(h)) return msg::PortValue::bytes(h.cast<std::string>());
    if (PyList_CheckExact(h.ptr()) && PyList_GET_SIZE(h.ptr()) > 0) {      // a plain list of token ids
        const Py_ssize_t n = PyList_GET_SIZE(h.ptr());
        std::vector<int32_t> ids(static_cast<size_t>(n));
        bool all_ids = true;
        for (Py_ssize_t i = 0; i < n && all_ids; ++i) {
            PyObject* item = PyList_GET_ITEM(h.ptr(), i);
            int overflow = 0;
            const long v = PyLong_CheckExact(item) ? PyLong_AsLongAndOverflow(item, &overflow) : 0;
            all_ids = PyLong_CheckExact(item) && !overflow && v >= INT32_MIN && v <= INT32_MAX;
            ids[static_cast<size_t>(i)] = static_cast<int32_t>(v);
        }
        if (all_ids) return msg::PortValue::token_ids(std::move(ids));
    }
    auto* held = new py::object(py::reinterpret_borrow<py::object>(h));
    return msg::PortValue::object(std::shared_ptr<void>(held, [](void* p) {
        py::gil_scoped_acquire gil;
        delete static_cast<py::object*>(p);
    }));
}

static py::object port_to_python(const msg::PortValue& v) {
    switch (v.kind) {
        case msg::PortValue::Kind::kText: return py::str(v.data);
        case msg::PortValue::Kind::kBytes: return py::bytes(v.data);
        case msg::PortValue::Kind::kTokens: return py::cast(v.tokens);
        case msg::PortValue::Kind::kFloats: {
            py::array_t<float> a(static_cast<py::ssize_t>(v.values.size()), v.values.data());
            return v.shape.empty() ? py::object(a) : py::object(a.attr("reshape")(py::cast(v.shape)));
        }
        case msg::PortValue::Kind::kOpaque: return *static_cast<py::object*>(v.opaque.get());
        default: return py::none();
    }
}

static msg::PortMap port_map_from_python(const py::dict& d) {
    msg::PortMap m;
    for (auto kv : d) {
        msg::PortValue v = port_from_python(kv.second);
        if (v.present()) m[kv.first.cast<std::string>()] = std::move(v);
    }
    return m;
}

static py::dict port_map_to_python(const msg::PortMap& m) {
    py::dict d;
    for (const auto& kv : m) d[py::str(kv.first)] = port_to_python(kv.second);
    return d;
}

// A Python callable ``fn(spec, batch: list[dict]) -> list[dict]`` as a native stage.
static msg::StageFn stage_fn_from_python(py::object fn) {
    auto held = std::shared_ptr<py::object>(new py::object(std::move(fn)), [](py::object* p) {
        py::gil_scoped_acquire gil;
        delete p;
    });
    return [held](const msg::StageSpec& spec, const std::vector<msg::PortMap>& batch) {
        py::gil_scoped_acquire gil;
        py::list in;
        for (const auto& m : batch) in.append(port_map_to_python(m));
        py::object out = (*held)(spec, in);
        std::vector<msg::PortMap> res;
        for (auto item : out) res.push_back(port_map_from_python(item.cast<py::dict>()));
        return res;
    };
}

struct MultiStageOutput {
    std::string text, stages, audio_pcm16;
    std::vector<int32_t> token_ids;
    int audio_sample_rate = 0, audio_channels = 0;
};

PYBIND11_MODULE(_telb_runtime, m) {
    m.doc() = "Native runtime of the B200 Edge-LLM framework: paged KV bookkeeping, scheduler, streaming, tokenizer";

    // ---- paged KV ------------------------------------------------------------------------------
    py::class_<PageAllocator>(m, "PageAllocator")
        .def(py::init<int>())
        .def_property_readonly("free_pages", &PageAllocator::free_pages)
        .def_property_readonly("num_pages", &PageAllocator::num_pages)
        .def("alloc", &PageAllocator::alloc)
        .def("retain", &PageAllocator::retain)
        .def("release", &PageAllocator::release)
        .def("refcount", &PageAllocator::refcount);
    py::class_<KVPageTable>(m, "KVPageTable")
        .def(py::init<int, int, int, int>(), py::arg("num_pages"), py::arg("page_size"), py::arg("max_seats"),
             py::arg("max_pages_per_seq"))
        .def_property_readonly("page_size", &KVPageTable::page_size)
        .def_property_readonly("max_seats", &KVPageTable::max_seats)
        .def_property_readonly("max_pages_per_seq", &KVPageTable::max_pages_per_seq)
        .def_property_readonly("free_pages", &KVPageTable::free_pages)
        .def("length", &KVPageTable::length)
        .def("capacity_tokens", &KVPageTable::capacity_tokens)
        .def("pages", &KVPageTable::pages)
        .def("reserve", &KVPageTable::reserve)
        .def("can_reserve", &KVPageTable::can_reserve)
        .def("adopt_prefix", &KVPageTable::adopt_prefix)
        .def("commit", &KVPageTable::commit)
        .def("rewind", &KVPageTable::rewind)
        .def("free_seat", &KVPageTable::free_seat)
        .def("retire_before", &KVPageTable::retire_before)
        .def("live_pages", &KVPageTable::live_pages)
        .def("take_dirty_rows", &KVPageTable::take_dirty_rows)
        .def("allocator", &KVPageTable::allocator, py::return_value_policy::reference_internal)
        .def("rows", [](const KVPageTable& t, const std::vector<int>& seats) {
            py::array_t<int32_t> out({static_cast<py::ssize_t>(seats.size()), static_cast<py::ssize_t>(t.max_pages_per_seq())});
            auto o = out.mutable_unchecked<2>();
            for (size_t i = 0; i < seats.size(); ++i) {
                const int32_t* r = t.row(seats[i]);
                for (int j = 0; j < t.max_pages_per_seq(); ++j) o(i, j) = r[j];
            }
            return out;
        });
    py::class_<ResidentSlotPool>(m, "ResidentSlotPool")
        .def(py::init<int>())
        .def("acquire", &ResidentSlotPool::acquire)
        .def("release", &ResidentSlotPool::release)
        .def("epoch", &ResidentSlotPool::epoch)
        .def_property_readonly("in_use", &ResidentSlotPool::in_use)
        .def_property_readonly("capacity", &ResidentSlotPool::capacity);
    py::class_<PrefixCache::Match>(m, "PrefixMatch")
        .def_readonly("pages", &PrefixCache::Match::pages)
        .def_readonly("tokens", &PrefixCache::Match::tokens);
    py::class_<PrefixCache::EvictionPlan>(m, "EvictionPlan")
        .def_readonly("pages_wanted", &PrefixCache::EvictionPlan::pages_wanted)
        .def_readonly("reclaimable_pages", &PrefixCache::EvictionPlan::reclaimable_pages)
        .def_readonly("pinned_skipped", &PrefixCache::EvictionPlan::pinned_skipped)
        .def_readonly("satisfied", &PrefixCache::EvictionPlan::satisfied)
        .def_readonly("victims", &PrefixCache::EvictionPlan::victims);
    py::class_<PrefixCache>(m, "PrefixCache")
        .def(py::init<PageAllocator&, int, int>(), py::arg("allocator"), py::arg("page_size"), py::arg("max_records") = 1024,
             py::keep_alive<1, 2>())
        .def("lookup", &PrefixCache::lookup, py::arg("tokens"), py::arg("seed") = 0)
        .def("insert", &PrefixCache::insert, py::arg("tokens"), py::arg("filled_tokens"), py::arg("pages"), py::arg("seed") = 0)
        .def_property_readonly("check_mismatches", &PrefixCache::check_mismatches)
        .def_static("extras_seed", &PrefixCache::extras_seed, py::arg("adapter") = "", py::arg("adapter_generation") = 0,
                    py::arg("isolation_key") = "")
        .def("evict", [](PrefixCache& c, int pages_wanted) { return c.evict(pages_wanted); })
        .def("evict_plan", [](PrefixCache& c, const PrefixCache::EvictionPlan& p) { return c.evict(p); })
        .def("plan_eviction", &PrefixCache::plan_eviction)
        .def("drop_records", &PrefixCache::drop_records)
        .def_property_readonly("records", &PrefixCache::records)
        .def_property_readonly("hits", &PrefixCache::hits)
        .def_property_readonly("misses", &PrefixCache::misses)
        .def_static("hash_block", [](uint64_t parent, const std::vector<int32_t>& toks) {
            return PrefixCache::hash_block(parent, toks.data(), static_cast<int>(toks.size()));
        });

    // ---- streaming -----------------------------------------------------------------------------
    py::enum_<FinishReason>(m, "FinishReason")
        .value("NotFinished", FinishReason::kNotFinished)
        .value("EndId", FinishReason::kEndId)
        .value("Length", FinishReason::kLength)
        .value("Cancelled", FinishReason::kCancelled)
        .value("Error", FinishReason::kError)
        .value("StopWords", FinishReason::kStopWords);
    py::class_<TokenLogprobs>(m, "TokenLogprobs")
        .def(py::init<>())
        .def_readwrite("chosen", &TokenLogprobs::chosen)
        .def_readwrite("top_ids", &TokenLogprobs::top_ids)
        .def_readwrite("top_values", &TokenLogprobs::top_values);
    py::class_<StreamChunk>(m, "StreamChunk")
        .def(py::init<>())
        .def_readwrite("token_ids", &StreamChunk::token_ids)
        .def_readwrite("logprobs", &StreamChunk::logprobs)
        .def_readwrite("text", &StreamChunk::text)
        .def_readwrite("finished", &StreamChunk::finished)
        .def_readwrite("reason", &StreamChunk::reason);
    py::class_<GenerationMetrics>(m, "GenerationMetrics")
        .def_readonly("generated_tokens", &GenerationMetrics::generated_tokens)
        .def_readonly("time_to_first_token_s", &GenerationMetrics::time_to_first_token_s)
        .def_readonly("generation_time_s", &GenerationMetrics::generation_time_s)
        .def_property_readonly("decode_tokens_per_second", &GenerationMetrics::decode_tokens_per_second);
    py::class_<StreamChannel, std::shared_ptr<StreamChannel>>(m, "StreamChannel")
        .def_static("create", &StreamChannel::create, py::arg("collect_metrics") = false)
        .def("push", &StreamChannel::push, py::arg("tokens"), py::arg("logprobs") = TokenLogprobs())
        .def("finish", &StreamChannel::finish)
        .def("try_pop", [](StreamChannel& c) -> py::object {
            StreamChunk ch;
            if (!c.try_pop(ch)) return py::none();
            return py::cast(ch);
        })
        .def("wait_pop", [](StreamChannel& c, double timeout_s) -> py::object {
            StreamChunk ch;
            bool ok;
            {
                py::gil_scoped_release rel;
                ok = c.wait_pop(ch, timeout_s);
            }
            if (!ok) return py::none();
            return py::cast(ch);
        }, py::arg("timeout_s") = 1.0)
        .def("cancel", &StreamChannel::cancel)
        .def_property_readonly("cancelled", &StreamChannel::cancelled)
        .def("is_finished", &StreamChannel::is_finished)
        .def("get_reason", &StreamChannel::reason)
        .def("set_stream_interval", &StreamChannel::set_stream_interval)
        .def("metrics", &StreamChannel::metrics);
    m.def("utf8_complete_prefix", [](const py::bytes& b) { return utf8_complete_prefix(std::string(b)); });

    // ---- scheduling ----------------------------------------------------------------------------
    py::enum_<IfbSchedulingMode>(m, "IfbSchedulingMode")
        .value("Auto", IfbSchedulingMode::kAuto).value("Mixed", IfbSchedulingMode::kMixed)
        .value("PrefillFirst", IfbSchedulingMode::kPrefillFirst).value("SingleCohort", IfbSchedulingMode::kSingleCohort);
    py::enum_<SchedulingPolicy>(m, "SchedulingPolicy").value("Fcfs", SchedulingPolicy::kFcfs).value("Priority", SchedulingPolicy::kPriority);
    py::enum_<PreemptionMode>(m, "PreemptionMode").value("NoPreemption", PreemptionMode::kNone).value("Pause", PreemptionMode::kPause);
    py::enum_<WorkKind>(m, "WorkKind").value("Context", WorkKind::kContext).value("Decode", WorkKind::kDecode);
    py::class_<SchedulingOptions>(m, "SchedulingOptions")
        .def(py::init<>())
        .def_readwrite("mode", &SchedulingOptions::mode)
        .def_readwrite("policy", &SchedulingOptions::policy)
        .def_readwrite("preemption", &SchedulingOptions::preemption)
        .def_readwrite("max_num_tokens", &SchedulingOptions::max_num_tokens)
        .def_readwrite("max_chunk_tokens", &SchedulingOptions::max_chunk_tokens)
        .def_readwrite("priority_reserved_slots", &SchedulingOptions::priority_reserved_slots)
        .def_readwrite("max_pause_steps", &SchedulingOptions::max_pause_steps)
        .def_readwrite("min_request_priority", &SchedulingOptions::min_request_priority);
    py::class_<SessionCapabilities>(m, "SessionCapabilities")
        .def(py::init<>())
        .def_readwrite("compact", &SessionCapabilities::compact)
        .def_readwrite("max_batch_size", &SessionCapabilities::max_batch_size)
        .def_readwrite("max_input_length", &SessionCapabilities::max_input_length)
        .def_readwrite("kv_page_size", &SessionCapabilities::kv_page_size)
        .def_readwrite("max_kv_tokens", &SessionCapabilities::max_kv_tokens);
    py::class_<ResolvedSchedulingPolicy>(m, "ResolvedSchedulingPolicy")
        .def(py::init<>())
        .def_readwrite("mode", &ResolvedSchedulingPolicy::mode)
        .def_readwrite("policy", &ResolvedSchedulingPolicy::policy)
        .def_readwrite("preemption", &ResolvedSchedulingPolicy::preemption)
        .def_readwrite("max_num_tokens", &ResolvedSchedulingPolicy::max_num_tokens)
        .def_readwrite("max_chunk_tokens", &ResolvedSchedulingPolicy::max_chunk_tokens)
        .def_readwrite("priority_reserved_slots", &ResolvedSchedulingPolicy::priority_reserved_slots)
        .def_readwrite("max_pause_steps", &ResolvedSchedulingPolicy::max_pause_steps);
    m.def("validate_scheduling_options", &validate_scheduling_options);
    m.def("resolve_scheduling_policy", &resolve_scheduling_policy);
    py::class_<ResidentState>(m, "ResidentState")
        .def(py::init<>())
        .def_readwrite("slot", &ResidentState::slot)
        .def_readwrite("epoch", &ResidentState::epoch)
        .def_readwrite("prompt_len", &ResidentState::prompt_len)
        .def_readwrite("prefilled", &ResidentState::prefilled)
        .def_readwrite("generated", &ResidentState::generated)
        .def_readwrite("priority", &ResidentState::priority)
        .def_readwrite("arrival", &ResidentState::arrival)
        .def_readwrite("paused_steps", &ResidentState::paused_steps)
        .def_readwrite("exclusive", &ResidentState::exclusive);
    py::class_<StepPlannerLimits>(m, "StepPlannerLimits")
        .def(py::init<>())
        .def_readwrite("max_batch_size", &StepPlannerLimits::max_batch_size)
        .def_readwrite("max_input_length", &StepPlannerLimits::max_input_length)
        .def_readwrite("kv_page_size", &StepPlannerLimits::kv_page_size);
    py::class_<PlannedSequence>(m, "PlannedSequence")
        .def(py::init<>())
        .def_readwrite("slot", &PlannedSequence::slot)
        .def_readwrite("epoch", &PlannedSequence::epoch)
        .def_readwrite("kind", &PlannedSequence::kind)
        .def_readwrite("start", &PlannedSequence::start)
        .def_readwrite("length", &PlannedSequence::length)
        .def_readwrite("last_chunk", &PlannedSequence::last_chunk);
    py::class_<StepPlan>(m, "StepPlan")
        .def(py::init<>())
        .def_readwrite("seqs", &StepPlan::seqs)
        .def_readwrite("paused", &StepPlan::paused)
        .def_readwrite("num_context", &StepPlan::num_context)
        .def_readwrite("num_decode", &StepPlan::num_decode)
        .def_readwrite("total_tokens", &StepPlan::total_tokens)
        .def("empty", &StepPlan::empty);
    py::class_<StepPlanner>(m, "StepPlanner")
        .def(py::init<StepPlannerLimits, ResolvedSchedulingPolicy>())
        .def("plan", &StepPlanner::plan);

    py::class_<GenerationRequest>(m, "GenerationRequest")
        .def(py::init<>())
        .def_readwrite("prompt_ids", &GenerationRequest::prompt_ids)
        .def_readwrite("max_tokens", &GenerationRequest::max_tokens)
        .def_readwrite("temperature", &GenerationRequest::temperature)
        .def_readwrite("top_k", &GenerationRequest::top_k)
        .def_readwrite("top_p", &GenerationRequest::top_p)
        .def_readwrite("seed", &GenerationRequest::seed)
        .def_readwrite("ignore_eos", &GenerationRequest::ignore_eos)
        .def_readwrite("stop_token_ids", &GenerationRequest::stop_token_ids)
        .def_readwrite("priority", &GenerationRequest::priority)
        .def_readwrite("exclusive", &GenerationRequest::exclusive)
        .def_readwrite("lora_name", &GenerationRequest::lora_name)
        .def_readwrite("stream_interval", &GenerationRequest::stream_interval)
        .def_readwrite("num_logprobs", &GenerationRequest::num_logprobs)
        .def_readwrite("guided_type", &GenerationRequest::guided_type)
        .def_readwrite("guided_spec", &GenerationRequest::guided_spec)
        .def_readwrite("logit_bias_ids", &GenerationRequest::logit_bias_ids)
        .def_readwrite("logit_bias_values", &GenerationRequest::logit_bias_values)
        .def_readwrite("cache_lookup", &GenerationRequest::cache_lookup)
        .def_readwrite("cache_commit", &GenerationRequest::cache_commit)
        .def_readwrite("disable_spec_decode", &GenerationRequest::disable_spec_decode)
        .def_readwrite("embeds_key", &GenerationRequest::embeds_key);
    py::class_<AdmissionResult>(m, "AdmissionResult")
        .def(py::init<>())
        .def_readwrite("admitted", &AdmissionResult::admitted)
        .def_readwrite("slot", &AdmissionResult::slot)
        .def_readwrite("reused_tokens", &AdmissionResult::reused_tokens)
        .def_readwrite("reason", &AdmissionResult::reason)
        .def_readwrite("retry_later", &AdmissionResult::retry_later);
    py::class_<TokenDelta>(m, "TokenDelta")
        .def(py::init<>())
        .def_readwrite("slot", &TokenDelta::slot)
        .def_readwrite("tokens", &TokenDelta::tokens)
        .def_readwrite("logprobs", &TokenDelta::logprobs)
        .def_readwrite("finished", &TokenDelta::finished)
        .def_readwrite("reason", &TokenDelta::reason);
    py::class_<StepResult>(m, "StepResult").def(py::init<>()).def_readwrite("deltas", &StepResult::deltas);
    py::register_exception<SessionLostError>(m, "SessionLostError");
    py::class_<RuntimeSession, PyRuntimeSession, std::shared_ptr<RuntimeSession>>(m, "RuntimeSession")
        .def(py::init<>())
        .def("capabilities", &RuntimeSession::capabilities)
        .def("admit", &RuntimeSession::admit)
        .def("execute", &RuntimeSession::execute)
        .def("release", &RuntimeSession::release);

    py::class_<EngineConfig>(m, "EngineConfig")
        .def(py::init<>())
        .def_readwrite("command_queue_capacity", &EngineConfig::command_queue_capacity)
        .def_readwrite("max_pending_requests", &EngineConfig::max_pending_requests)
        .def_readwrite("max_batch_size", &EngineConfig::max_batch_size)
        .def_readwrite("max_consecutive_session_failures", &EngineConfig::max_consecutive_session_failures)
        .def_readwrite("idle_wait_s", &EngineConfig::idle_wait_s)
        .def_readwrite("scheduling", &EngineConfig::scheduling);
    py::class_<EngineMetrics>(m, "EngineMetrics")
        .def_readonly("submitted", &EngineMetrics::submitted).def_readonly("refused", &EngineMetrics::refused)
        .def_readonly("completed", &EngineMetrics::completed).def_readonly("cancelled", &EngineMetrics::cancelled)
        .def_readonly("failed", &EngineMetrics::failed).def_readonly("admitted_mid_flight", &EngineMetrics::admitted_mid_flight)
        .def_readonly("stalls_no_capacity", &EngineMetrics::stalls_no_capacity)
        .def_readonly("stalls_exclusive", &EngineMetrics::stalls_exclusive)
        .def_readonly("decode_steps", &EngineMetrics::decode_steps).def_readonly("prompt_steps", &EngineMetrics::prompt_steps)
        .def_readonly("mixed_steps", &EngineMetrics::mixed_steps).def_readonly("step_tokens", &EngineMetrics::step_tokens)
        .def_readonly("paused_resident_steps", &EngineMetrics::paused_resident_steps)
        .def_readonly("session_failures", &EngineMetrics::session_failures)
        .def_readonly("prefix_reused_tokens", &EngineMetrics::prefix_reused_tokens)
        .def_readonly("queue_latency_s_sum", &EngineMetrics::queue_latency_s_sum);
    py::class_<EngineStatus>(m, "EngineStatus")
        .def_readonly("available", &EngineStatus::available)
        .def_readonly("unavailable_reason", &EngineStatus::unavailable_reason)
        .def_readonly("queued", &EngineStatus::queued)
        .def_readonly("resident", &EngineStatus::resident);
    py::class_<RequestStats>(m, "RequestStats")
        .def_readonly("prompt_tokens", &RequestStats::prompt_tokens)
        .def_readonly("generated_tokens", &RequestStats::generated_tokens)
        .def_readonly("reused_tokens", &RequestStats::reused_tokens)
        .def_readonly("queue_s", &RequestStats::queue_s).def_readonly("ttft_s", &RequestStats::ttft_s)
        .def_readonly("total_s", &RequestStats::total_s);
    py::class_<RequestHandle, std::shared_ptr<RequestHandle>>(m, "RequestHandle")
        .def_property_readonly("id", &RequestHandle::id)
        .def("stream", &RequestHandle::stream)
        .def("ready", &RequestHandle::ready)
        .def("get", [](RequestHandle& h, double timeout_s) {
            py::gil_scoped_release rel;
            return h.get(timeout_s);
        }, py::arg("timeout_s") = 1e9)
        .def("logprobs", &RequestHandle::logprobs)
        .def("reason", &RequestHandle::reason)
        .def("error", &RequestHandle::error)
        .def("cancel", &RequestHandle::cancel)
        .def("stats", &RequestHandle::stats);
    py::class_<RequestEngine>(m, "RequestEngine")
        .def(py::init([](EngineConfig cfg, py::function factory) {
            SessionFactory f = session_factory_from_python(std::move(factory));
            py::gil_scoped_release rel;       // the constructor opens the first session on this thread, then starts the actor
            return new RequestEngine(cfg, f);
        }))
        .def("submit", [](RequestEngine& e, const GenerationRequest& r) {
            std::string why;
            auto h = e.submit(r, &why);
            return py::make_tuple(h, why);
        })
        .def("cancel", &RequestEngine::cancel)
        .def("shutdown", [](RequestEngine& e) {
            py::gil_scoped_release rel;
            e.shutdown();
        })
        .def("queued", &RequestEngine::queued)
        .def("resident", &RequestEngine::resident)
        .def("metrics", &RequestEngine::metrics)
        .def("status", &RequestEngine::status)
        .def("resolved_policy", &RequestEngine::resolved_policy);

    // ---- ragged batch / sampling / config / misc ------------------------------------------------
    py::class_<RaggedBatch>(m, "RaggedBatch")
        .def_readonly("q_start", &RaggedBatch::q_start).def_readonly("q_len", &RaggedBatch::q_len)
        .def_readonly("past_len", &RaggedBatch::past_len).def_readonly("positions", &RaggedBatch::positions)
        .def_readonly("seq_ids", &RaggedBatch::seq_ids).def_readonly("slot_ids", &RaggedBatch::slot_ids)
        .def_readonly("logits_idx", &RaggedBatch::logits_idx).def_readonly("num_seqs", &RaggedBatch::num_seqs)
        .def_readonly("num_tokens", &RaggedBatch::num_tokens).def_readonly("max_q_len", &RaggedBatch::max_q_len)
        .def_readonly("max_seq_len", &RaggedBatch::max_seq_len);
    m.def("build_ragged_batch", &RaggedBatchBuilder::build, py::arg("plan"), py::arg("past_lens"), py::arg("logits_all") = false);
    py::class_<RowSamplingParams>(m, "RowSamplingParams")
        .def(py::init<>())
        .def_readwrite("temperature", &RowSamplingParams::temperature)
        .def_readwrite("top_k", &RowSamplingParams::top_k)
        .def_readwrite("top_p", &RowSamplingParams::top_p)
        .def("greedy", &RowSamplingParams::greedy);
    m.def("request_stable_uniform", &request_stable_uniform);
    m.def("sample_row", [](py::array_t<float, py::array::c_style | py::array::forcecast> logits, const RowSamplingParams& p, float u) {
        return sample_row(logits.data(), static_cast<int>(logits.size()), p, u);
    });
    py::class_<ParallelConfig>(m, "ParallelConfig")
        .def(py::init<>())
        .def_readwrite("world_size", &ParallelConfig::world_size)
        .def_readwrite("rank", &ParallelConfig::rank)
        .def_readwrite("launch_mode", &ParallelConfig::launch_mode)
        .def("validate", &ParallelConfig::validate);
    py::class_<LLMEngineConfig>(m, "LLMEngineConfig")
        .def(py::init<>())
        .def_static("from_json", [](const std::string& text) { return LLMEngineConfig::from_json(Json::parse(text)); })
        .def("to_json", [](const LLMEngineConfig& c) { return c.to_json().dump(); })
        .def_readwrite("model_type", &LLMEngineConfig::model_type)
        .def_readwrite("vocab_size", &LLMEngineConfig::vocab_size)
        .def_readwrite("hidden_size", &LLMEngineConfig::hidden_size)
        .def_readwrite("num_layers", &LLMEngineConfig::num_layers)
        .def_readwrite("num_heads", &LLMEngineConfig::num_heads)
        .def_readwrite("num_kv_heads", &LLMEngineConfig::num_kv_heads)
        .def_readwrite("head_dim", &LLMEngineConfig::head_dim)
        .def_readwrite("max_batch_size", &LLMEngineConfig::max_batch_size)
        .def_readwrite("max_input_len", &LLMEngineConfig::max_input_len)
        .def_readwrite("max_kv_cache_capacity", &LLMEngineConfig::max_kv_cache_capacity)
        .def_readwrite("kv_page_size", &LLMEngineConfig::kv_page_size)
        .def_readwrite("dtype", &LLMEngineConfig::dtype)
        .def_readwrite("quantization", &LLMEngineConfig::quantization)
        .def_readwrite("decoding_strategies", &LLMEngineConfig::decoding_strategies)
        .def_readwrite("world_size", &LLMEngineConfig::world_size)
        .def_static("from_runtime_config", [](const std::string& text) { return LLMEngineConfig::from_runtime_config(Json::parse(text)); })
        .def_readwrite("kv_cache_dtype", &LLMEngineConfig::kv_cache_dtype)
        .def_readwrite("intermediate_size", &LLMEngineConfig::intermediate_size)
        .def_readwrite("max_position_embeddings", &LLMEngineConfig::max_position_embeddings)
        .def_readwrite("rotary_dim", &LLMEngineConfig::rotary_dim)
        .def_readwrite("rms_norm_eps", &LLMEngineConfig::rms_norm_eps)
        .def_readwrite("rope_theta", &LLMEngineConfig::rope_theta)
        .def_readwrite("rope_scaling_type", &LLMEngineConfig::rope_scaling_type)
        .def_readwrite("rope_scaling_factor", &LLMEngineConfig::rope_scaling_factor)
        .def_readwrite("mrope_section", &LLMEngineConfig::mrope_section)
        .def_readwrite("has_qk_norm", &LLMEngineConfig::has_qk_norm)
        .def_readwrite("sliding_window", &LLMEngineConfig::sliding_window)
        .def_readwrite("layer_windows", &LLMEngineConfig::layer_windows)
        .def_readwrite("layer_types", &LLMEngineConfig::layer_types)
        .def_readwrite("mlp_types", &LLMEngineConfig::mlp_types)
        .def_readwrite("num_kv_shared_layers", &LLMEngineConfig::num_kv_shared_layers)
        .def_readwrite("num_experts", &LLMEngineConfig::num_experts)
        .def_readwrite("num_experts_per_tok", &LLMEngineConfig::num_experts_per_tok)
        .def_readwrite("moe_intermediate_size", &LLMEngineConfig::moe_intermediate_size)
        .def_readwrite("quant_group_size", &LLMEngineConfig::quant_group_size)
        .def_readwrite("draft_type", &LLMEngineConfig::draft_type)
        .def_readwrite("dflash_projector_type", &LLMEngineConfig::dflash_projector_type)
        .def_readwrite("dflash_block_size", &LLMEngineConfig::dflash_block_size)
        .def_readwrite("dflash_version", &LLMEngineConfig::dflash_version)
        .def_readwrite("draft_candidate_count", &LLMEngineConfig::draft_candidate_count)
        .def_readwrite("dspark_markov_rank", &LLMEngineConfig::dspark_markov_rank)
        .def_readwrite("is_diffusion", &LLMEngineConfig::is_diffusion)
        .def_readwrite("diffusion_canvas_length", &LLMEngineConfig::diffusion_canvas_length)
        .def_readwrite("eos_token_ids", &LLMEngineConfig::eos_token_ids)
        .def_readwrite("mamba_num_heads", &LLMEngineConfig::mamba_num_heads)
        .def_readwrite("mamba_d_state", &LLMEngineConfig::mamba_d_state)
        .def_readwrite("gdn_num_v_heads", &LLMEngineConfig::gdn_num_v_heads)
        .def("is_hybrid", &LLMEngineConfig::is_hybrid)
        .def("is_moe", &LLMEngineConfig::is_moe)
        .def("num_attention_layers", &LLMEngineConfig::num_attention_layers)
        .def("num_recurrent_layers", &LLMEngineConfig::num_recurrent_layers)
        .def("kv_bytes_per_token", &LLMEngineConfig::kv_bytes_per_token)
        .def("kv_pool_bytes", &LLMEngineConfig::kv_pool_bytes)
        .def("recurrent_state_bytes_per_seat", &LLMEngineConfig::recurrent_state_bytes_per_seat)
        .def("validate", &LLMEngineConfig::validate);
    py::class_<LoraAdapter>(m, "LoraAdapter")
        .def(py::init<>())
        .def_readwrite("name", &LoraAdapter::name).def_readwrite("path", &LoraAdapter::path)
        .def_readwrite("rank", &LoraAdapter::rank).def_readwrite("scale", &LoraAdapter::scale);
    py::class_<LoRAManager>(m, "LoRAManager")
        .def(py::init<>())
        .def("add", &LoRAManager::add).def("remove", &LoRAManager::remove)
        .def("find", &LoRAManager::find, py::return_value_policy::reference_internal)
        .def("activate", &LoRAManager::activate)
        .def("active", &LoRAManager::active, py::return_value_policy::reference_internal)
        .def("names", &LoRAManager::names);
    py::class_<DeviceFailureState>(m, "DeviceFailureState")
        .def(py::init<>())
        .def("record", &DeviceFailureState::record)
        .def("failed", &DeviceFailureState::failed)
        .def("reason", &DeviceFailureState::reason);
    py::class_<StageTimer>(m, "StageTimer")
        .def(py::init<>())
        .def("set_enabled", &StageTimer::set_enabled)
        .def("begin", &StageTimer::begin)
        .def("end", &StageTimer::end)
        .def("reset", &StageTimer::reset)
        .def("snapshot", [](const StageTimer& t) {
            py::dict d;
            for (const auto& kv : t.snapshot())
                d[py::str(kv.first)] = py::make_tuple(kv.second.count, kv.second.total_s, kv.second.max_s);
            return d;
        });
    m.def("json_roundtrip", [](const std::string& s) { return Json::parse(s).dump(); });

    // ---- tokenizer -----------------------------------------------------------------------------
    py::class_<Tokenizer>(m, "Tokenizer")
        .def_static("load_from_hf", &Tokenizer::load_from_hf)
        .def_static("from_json_text", &Tokenizer::from_json_text, py::arg("tokenizer_json"), py::arg("config_json") = "")
        .def("encode", &Tokenizer::encode, py::arg("text"), py::arg("add_special_tokens") = false)
        .def("decode", [](const Tokenizer& t, const std::vector<int32_t>& ids, bool skip) { return py::bytes(t.decode(ids, skip)); },
             py::arg("ids"), py::arg("skip_special_tokens") = true)
        .def("id_to_bytes", [](const Tokenizer& t, int32_t id) { return py::bytes(t.id_to_bytes(id)); })
        .def("id_to_piece", &Tokenizer::id_to_piece)
        .def("piece_to_id", &Tokenizer::piece_to_id)
        .def_property_readonly("vocab_size", &Tokenizer::vocab_size)
        .def_property_readonly("bos_id", &Tokenizer::bos_id)
        .def_property_readonly("eos_id", &Tokenizer::eos_id)
        .def("is_special", &Tokenizer::is_special);
    py::class_<ChatMessage>(m, "ChatMessage")
        .def(py::init<>())
        .def(py::init([](const std::string& r, const std::string& c) { return ChatMessage{r, c}; }))
        .def_readwrite("role", &ChatMessage::role)
        .def_readwrite("content", &ChatMessage::content);
    py::class_<ChatTemplate>(m, "ChatTemplate")
        .def_static("load", &ChatTemplate::load)
        .def_static("from_template_text", &ChatTemplate::from_template_text, py::arg("template"), py::arg("bos") = "")
        .def("apply", &ChatTemplate::apply, py::arg("messages"), py::arg("add_generation_prompt") = true,
             py::arg("enable_thinking") = true);
    // ---- media ---------------------------------------------------------------------------------
    py::class_<AudioClip>(m, "AudioClip")
        .def_readonly("sample_rate", &AudioClip::sample_rate)
        .def_property_readonly("samples", [](const AudioClip& c) { return py::array_t<float>(c.samples.size(), c.samples.data()); });
    m.def("parse_wav", [](py::bytes b) { return parse_wav(std::string(b)); });
    m.def("load_wav", &load_wav);
    m.def("parse_flac", [](py::bytes b) { return parse_flac(std::string(b)); });
    m.def("parse_audio", [](py::bytes b) { return parse_audio(std::string(b)); });
    m.def("load_audio", &load_audio);
    m.def("resample_linear", [](py::array_t<float, py::array::c_style | py::array::forcecast> x, int from_rate, int to_rate) {
        std::vector<float> v(x.data(), x.data() + x.size());
        const auto y = resample_linear(v, from_rate, to_rate);
        return py::array_t<float>(y.size(), y.data());
    });
    py::class_<MelConfig>(m, "MelConfig")
        .def(py::init<>())
        .def_readwrite("sample_rate", &MelConfig::sample_rate)
        .def_readwrite("n_fft", &MelConfig::n_fft)
        .def_readwrite("hop", &MelConfig::hop)
        .def_readwrite("n_mels", &MelConfig::n_mels)
        .def_readwrite("f_min", &MelConfig::f_min)
        .def_readwrite("f_max", &MelConfig::f_max)
        .def_readwrite("whisper_norm", &MelConfig::whisper_norm)
        .def_readwrite("pad_to_samples", &MelConfig::pad_to_samples);
    m.def("mel_filterbank", [](const MelConfig& c) {
        const auto fb = mel_filterbank(c);
        py::array_t<float> out({static_cast<py::ssize_t>(c.n_mels), static_cast<py::ssize_t>(c.n_fft / 2 + 1)});
        std::copy(fb.begin(), fb.end(), out.mutable_data());
        return out;
    });
    m.def("log_mel_spectrogram", [](py::array_t<float, py::array::c_style | py::array::forcecast> x, const MelConfig& c) {
        std::vector<float> v(x.data(), x.data() + x.size());
        int frames = 0;
        std::vector<float> mel;
        {
            py::gil_scoped_release rel;
            mel = log_mel_spectrogram(v, c, &frames);
        }
        py::array_t<float> out({static_cast<py::ssize_t>(c.n_mels), static_cast<py::ssize_t>(frames)});
        std::copy(mel.begin(), mel.end(), out.mutable_data());
        return out;
    });
    py::class_<Image>(m, "Image")
        .def_readonly("width", &Image::width)
        .def_readonly("height", &Image::height)
        .def_readonly("channels", &Image::channels)
        .def_property_readonly("pixels", [](const Image& im) {
            py::array_t<uint8_t> out({static_cast<py::ssize_t>(im.height), static_cast<py::ssize_t>(im.width), static_cast<py::ssize_t>(im.channels)});
            std::copy(im.pixels.begin(), im.pixels.end(), out.mutable_data());
            return out;
        });
    m.def("parse_image", [](py::bytes b) { return parse_image(std::string(b)); });
    m.def("load_image", &load_image);
    m.def("decode_png", [](py::bytes b) { return decode_png(std::string(b)); });
    m.def("decode_jpeg", [](py::bytes b) { return decode_jpeg(std::string(b)); });
    m.def("inflate_zlib", [](py::bytes b, size_t max_output) { return py::bytes(inflate_zlib(std::string(b), max_output)); },
          py::arg("stream"), py::arg("max_output") = size_t(1) << 30);
    m.def("image_from_array", [](py::array_t<uint8_t, py::array::c_style | py::array::forcecast> a) {
        if (a.ndim() != 3) throw std::runtime_error("expected an HWC uint8 array");
        Image im;
        im.height = static_cast<int>(a.shape(0));
        im.width = static_cast<int>(a.shape(1));
        im.channels = static_cast<int>(a.shape(2));
        im.pixels.assign(a.data(), a.data() + a.size());
        return im;
    });
    m.def("resize_bilinear", &resize_bilinear);
    m.def("resize_bicubic", &resize_bicubic);
    m.def("normalize_chw", [](const Image& im, const std::vector<float>& mean, const std::vector<float>& stddev) {
        const auto v = normalize_chw(im, mean, stddev);
        py::array_t<float> out({static_cast<py::ssize_t>(im.channels), static_cast<py::ssize_t>(im.height), static_cast<py::ssize_t>(im.width)});
        std::copy(v.begin(), v.end(), out.mutable_data());
        return out;
    });
    m.def("smart_resize", [](int h, int w, int factor, long long min_pixels, long long max_pixels) {
        int oh = 0, ow = 0;
        smart_resize(h, w, factor, min_pixels, max_pixels, &oh, &ow);
        return py::make_tuple(oh, ow);
    });
    // ---- per-layer-embedding store ---------------------------------------------------------------
    py::class_<PleTable>(m, "PleTable")
        .def(py::init<const std::string&>())
        .def_static("write", [](const std::string& path, py::array data, uint32_t layers, uint32_t dtype) {
            if (data.ndim() != 2 || !(data.flags() & py::array::c_style)) throw std::runtime_error("expected a C-contiguous 2-D array");
            PleTable::write(path, data.data(), static_cast<uint32_t>(data.shape(0)), static_cast<uint32_t>(data.shape(1) * data.itemsize()), layers, dtype);
        })
        .def_property_readonly("rows", &PleTable::rows)
        .def_property_readonly("row_bytes", &PleTable::row_bytes)
        .def_property_readonly("layers", &PleTable::layers)
        .def_property_readonly("dtype", &PleTable::dtype);
    py::class_<PleRun>(m, "PleRun")
        .def_readonly("first_row", &PleRun::first_row)
        .def_readonly("count", &PleRun::count)
        .def_readonly("staging_row", &PleRun::staging_row);
    py::class_<PleReadPlan>(m, "PleReadPlan")
        .def_readonly("slots", &PleReadPlan::slots)
        .def_readonly("miss_rows", &PleReadPlan::miss_rows)
        .def_readonly("miss_slots", &PleReadPlan::miss_slots)
        .def_readonly("runs", &PleReadPlan::runs)
        .def_readonly("hits", &PleReadPlan::hits)
        .def_readonly("misses", &PleReadPlan::misses)
        .def_readonly("deferred", &PleReadPlan::deferred)
        .def_readonly("bytes", &PleReadPlan::bytes);
    py::class_<PleIoBudget>(m, "PleIoBudget")
        .def(py::init<uint64_t, int>(), py::arg("bytes_per_step"), py::arg("burst_steps") = 2)
        .def("begin_step", &PleIoBudget::begin_step)
        .def("take", &PleIoBudget::take)
        .def_property_readonly("available", &PleIoBudget::available);
    py::class_<PleCache>(m, "PleCache")
        .def(py::init<int>())
        .def("plan", &PleCache::plan, py::arg("ids"), py::arg("row_bytes"), py::arg("budget") = nullptr)
        .def("lookup", &PleCache::lookup)
        .def_property_readonly("slots", &PleCache::slots)
        .def_property_readonly("hits", &PleCache::hits)
        .def_property_readonly("misses", &PleCache::misses);
    py::class_<PleReadExecutor>(m, "PleReadExecutor")
        .def(py::init<int>(), py::arg("threads") = 2)
        .def("read", [](PleReadExecutor& ex, const PleTable& t, const PleReadPlan& plan, uintptr_t staging) {
            py::gil_scoped_release rel;
            ex.read(t, plan, reinterpret_cast<uint8_t*>(staging));
        });

    // ---- the façade ----
    py::class_<LLMGenerationRequest::Entry>(m, "GenerationEntry")
        .def(py::init<>())
        .def_readwrite("messages", &LLMGenerationRequest::Entry::messages)
        .def_readwrite("prompt", &LLMGenerationRequest::Entry::prompt)
        .def_readwrite("prompt_ids", &LLMGenerationRequest::Entry::prompt_ids);
    py::class_<LLMGenerationRequest>(m, "LLMGenerationRequest")
        .def(py::init<>())
        .def_readwrite("requests", &LLMGenerationRequest::requests)
        .def_readwrite("max_generate_length", &LLMGenerationRequest::max_generate_length)
        .def_readwrite("temperature", &LLMGenerationRequest::temperature)
        .def_readwrite("top_k", &LLMGenerationRequest::top_k)
        .def_readwrite("top_p", &LLMGenerationRequest::top_p)
        .def_readwrite("seed", &LLMGenerationRequest::seed)
        .def_readwrite("apply_chat_template", &LLMGenerationRequest::apply_chat_template)
        .def_readwrite("add_generation_prompt", &LLMGenerationRequest::add_generation_prompt)
        .def_readwrite("enable_thinking", &LLMGenerationRequest::enable_thinking)
        .def_readwrite("ignore_eos", &LLMGenerationRequest::ignore_eos)
        .def_readwrite("stop", &LLMGenerationRequest::stop)
        .def_readwrite("stop_token_ids", &LLMGenerationRequest::stop_token_ids)
        .def_readwrite("lora_name", &LLMGenerationRequest::lora_name)
        .def_readwrite("num_logprobs", &LLMGenerationRequest::num_logprobs)
        .def_readwrite("priority", &LLMGenerationRequest::priority)
        .def_readwrite("disable_spec_decode", &LLMGenerationRequest::disable_spec_decode)
        .def_readwrite("cache_lookup", &LLMGenerationRequest::cache_lookup)
        .def_readwrite("cache_commit", &LLMGenerationRequest::cache_commit)
        .def_readwrite("timeout_s", &LLMGenerationRequest::timeout_s);
    py::class_<LLMGenerationResponse>(m, "LLMGenerationResponse")
        .def(py::init<>())
        .def_readonly("output_ids", &LLMGenerationResponse::output_ids)
        .def_property_readonly("output_texts", [](const LLMGenerationResponse& r) {
            py::list out;                                    // text cut by a length limit may end inside a UTF-8 sequence
            for (const auto& t : r.output_texts) out.append(py::reinterpret_steal<py::object>(PyUnicode_DecodeUTF8(t.data(), (Py_ssize_t)t.size(), "replace")));
            return out;
        })
        .def_readonly("finish_reasons", &LLMGenerationResponse::finish_reasons)
        .def_readonly("errors", &LLMGenerationResponse::errors)
        .def_readonly("stats", &LLMGenerationResponse::stats)
        .def_readonly("logprobs", &LLMGenerationResponse::logprobs);
    py::class_<LLMInferenceRuntime>(m, "LLMInferenceRuntime")
        .def(py::init([](EngineConfig cfg, py::function factory, const Tokenizer& tokenizer, py::object chat_template, bool has_draft_model,
                         py::object capture_hook) {
            RuntimeOptions opt;
            opt.engine = cfg;
            opt.has_draft_model = has_draft_model;
            if (!capture_hook.is_none()) {
                auto hook = std::make_shared<py::function>(capture_hook.cast<py::function>());
                opt.capture_hook = [hook]() {
                    py::gil_scoped_acquire gil;
                    return (*hook)().cast<bool>();
                };
            }
            std::shared_ptr<const ChatTemplate> tpl;
            if (!chat_template.is_none()) tpl = std::make_shared<ChatTemplate>(chat_template.cast<ChatTemplate>());
            SessionFactory f = session_factory_from_python(std::move(factory));
            auto tok = std::make_shared<Tokenizer>(tokenizer);
            py::gil_scoped_release rel;          // the engine opens its first session on this thread, then starts the actor
            return new LLMInferenceRuntime(std::move(opt), std::move(f), std::move(tok), std::move(tpl));
        }), py::arg("engine_config"), py::arg("session_factory"), py::arg("tokenizer"), py::arg("chat_template") = py::none(),
             py::arg("has_draft_model") = false, py::arg("capture_hook") = py::none())
        .def("handle_request", [](LLMInferenceRuntime& rt, const LLMGenerationRequest& req, py::object on_tokens) {
            LLMGenerationResponse resp;
            std::string err;
            StreamCallback cb;
            if (!on_tokens.is_none()) {
                auto fn = std::make_shared<py::function>(on_tokens.cast<py::function>());
                cb = [fn](int i, const std::vector<int32_t>& toks, const std::string& text, bool finished) {
                    py::gil_scoped_acquire gil;
                    (*fn)(i, toks, py::reinterpret_steal<py::object>(PyUnicode_DecodeUTF8(text.data(), (Py_ssize_t)text.size(), "replace")), finished);
                };
            }
            bool ok;
            {
                py::gil_scoped_release rel;
                ok = rt.handle_request(req, resp, cb, &err);
            }
            if (!ok) throw std::runtime_error(err);
            return resp;
        }, py::arg("request"), py::arg("on_tokens") = py::none())
        .def("build_prompt_ids", &LLMInferenceRuntime::build_prompt_ids)
        .def("count_prompt_tokens", &LLMInferenceRuntime::count_prompt_tokens)
        .def("capture_decoding_cuda_graph", [](LLMInferenceRuntime& rt) {
            py::gil_scoped_release rel;
            return rt.capture_decoding_cuda_graph();
        })
        .def("unavailable_reason", &LLMInferenceRuntime::unavailable_reason)
        .def("has_draft_model", &LLMInferenceRuntime::has_draft_model)
        .def("supports_seated_admission", &LLMInferenceRuntime::supports_seated_admission)
        .def("supports_stepped_execution", &LLMInferenceRuntime::supports_stepped_execution)
        .def("submit", [](LLMInferenceRuntime& rt, const GenerationRequest& r) {
            std::string why;
            auto h = rt.submit(r, &why);
            return py::make_tuple(h, why);
        })
        .def("open_session", [](LLMInferenceRuntime& rt) {
            std::shared_ptr<RuntimeSession> s;
            {
                py::gil_scoped_release rel;
                s = rt.open_session();
            }
            return s;
        })
        .def("metrics", &LLMInferenceRuntime::metrics)
        .def("queued", [](LLMInferenceRuntime& rt) { return rt.engine().queued(); })
        .def("resident", [](LLMInferenceRuntime& rt) { return rt.engine().resident(); })
        .def("status", [](LLMInferenceRuntime& rt) { return rt.engine().status(); })
        .def("cancel", [](LLMInferenceRuntime& rt, uint64_t id) { rt.engine().cancel(id); })
        .def("resolved_policy", [](LLMInferenceRuntime& rt) { return rt.engine().resolved_policy(); })
        .def("shutdown", [](LLMInferenceRuntime& rt) {
            py::gil_scoped_release rel;
            rt.shutdown();
        });

    // ---- stage graph ---------------------------------------------------------------------------------------------
    py::module_ ms = m.def_submodule("multistage", "Stage-graph runtime: config, validation, routes, cohorts, run loop");
    py::register_exception<msg::GraphError>(ms, "GraphError", PyExc_ValueError);
    ms.attr("SCHEMA_VERSION") = msg::kSchemaVersion;
    ms.attr("CONFIG_NAME") = msg::kConfigName;
    py::class_<msg::InputPort>(ms, "InputPort")
        .def_readonly("name", &msg::InputPort::name).def_readonly("source", &msg::InputPort::source)
        .def_readonly("on_missing", &msg::InputPort::on_missing)
        .def_property_readonly("from_request", &msg::InputPort::from_request)
        .def_property_readonly("ref", &msg::InputPort::ref);
    py::class_<msg::EmitPort>(ms, "EmitPort")
        .def_readonly("id", &msg::EmitPort::id).def_readonly("kind", &msg::EmitPort::kind)
        .def_readonly("transport", &msg::EmitPort::transport).def_readonly("terminal", &msg::EmitPort::terminal);
    py::class_<msg::StageSpec>(ms, "StageSpec")
        .def_readonly("id", &msg::StageSpec::id).def_readonly("runner", &msg::StageSpec::runner)
        .def_readonly("artifact", &msg::StageSpec::artifact).def_readonly("kind", &msg::StageSpec::kind)
        .def_readonly("inputs", &msg::StageSpec::inputs).def_readonly("emits", &msg::StageSpec::emits)
        .def_readonly("max_batch", &msg::StageSpec::max_batch).def_readonly("max_seq", &msg::StageSpec::max_seq)
        .def_property_readonly("config_json", [](const msg::StageSpec& s) { return s.config.dump(); });
    py::class_<msg::Route>(ms, "Route")
        .def_readonly("stages", &msg::Route::stages).def_readonly("terminals", &msg::Route::terminals)
        .def_property_readonly("skipped", [](const msg::Route& r) {
            py::dict d;
            for (const auto& kv : r.skipped) d[py::str(kv.first)] = kv.second;
            return d;
        })
        .def_property_readonly("error", [](const msg::Route& r) -> py::object { return r.error.empty() ? py::object(py::none()) : py::object(py::str(r.error)); });
    py::class_<msg::StageGraph>(ms, "StageGraph")
        .def_static("parse_text", &msg::StageGraph::parse_text, py::arg("text"), py::arg("root") = ".")
        .def_static("load", &msg::StageGraph::load)
        .def_readonly("stages", &msg::StageGraph::stages).def_readonly("terminals", &msg::StageGraph::terminals)
        .def_readonly("root", &msg::StageGraph::root)
        .def("stage", &msg::StageGraph::stage, py::return_value_policy::reference_internal)
        .def("validate", [](const msg::StageGraph& g, bool check_runners) { return g.validate(check_runners ? &msg::RunnerTable::global() : nullptr); },
             py::arg("check_runners") = true)
        .def("topological", &msg::StageGraph::topological)
        .def("to_json", [](const msg::StageGraph& g) { return g.to_json().dump(); });
    ms.def("register_runner", [](const std::string& name, const std::string& kind, std::vector<std::string> inputs, std::vector<std::string> emits,
                                 std::vector<std::string> required_config, bool batches) {
        msg::RunnerDecl d;
        d.name = name;
        d.kind = kind;
        d.inputs = std::move(inputs);
        d.emits = std::move(emits);
        d.required_config = std::move(required_config);
        d.batches = batches;
        msg::RunnerTable::global().add(std::move(d));
    }, py::arg("name"), py::arg("kind"), py::arg("inputs") = std::vector<std::string>(), py::arg("emits") = std::vector<std::string>(),
       py::arg("required_config") = std::vector<std::string>(), py::arg("batches") = true);
    ms.def("runner_names", [] { return msg::RunnerTable::global().names(); });
    ms.def("plan_route", [](const msg::StageGraph& g, const std::set<std::string>& fields, py::object want) {
        if (want.is_none()) return msg::plan_route(g, fields, nullptr);
        const auto w = want.cast<std::vector<std::string>>();
        return msg::plan_route(g, fields, &w);
    }, py::arg("graph"), py::arg("fields"), py::arg("want") = py::none());
    py::class_<msg::StageResponse>(ms, "StageResponse")
        .def_readonly("ok", &msg::StageResponse::ok)
        .def_property_readonly("error", [](const msg::StageResponse& r) -> py::object { return r.ok ? py::object(py::none()) : py::object(py::str(r.error)); })
        .def_property_readonly("outputs", [](const msg::StageResponse& r) {
            py::dict d;
            for (const auto& kv : r.outputs) d[py::str(kv.first)] = port_to_python(kv.second);
            return d;
        })
        .def_property_readonly("stages_json", [](const msg::StageResponse& r) { return r.diagnostics().dump(); });
    py::class_<MultiStageOutput>(ms, "MultiStageOutput")
        .def_readonly("text", &MultiStageOutput::text).def_readonly("stages", &MultiStageOutput::stages)
        .def_readonly("token_ids", &MultiStageOutput::token_ids)
        .def_property_readonly("audio_pcm16", [](const MultiStageOutput& o) { return py::bytes(o.audio_pcm16); })
        .def_readonly("audio_sample_rate", &MultiStageOutput::audio_sample_rate)
        .def_readonly("audio_channels", &MultiStageOutput::audio_channels);
    py::class_<msg::MultiStageRuntime>(ms, "MultiStageRuntime", "Runs requests through the stage graph of an engine directory")
        .def(py::init<>())
        .def(py::init([](const std::string& config_dir) {
            auto rt = std::make_unique<msg::MultiStageRuntime>();
            rt->load_dir(config_dir);
            return rt;
        }), py::arg("config_dir"))
        .def("load", &msg::MultiStageRuntime::load, py::arg("graph"), py::arg("check_runners") = true)
        .def("load_dir", &msg::MultiStageRuntime::load_dir, py::arg("path"), py::arg("check_runners") = true)
        .def_property_readonly("graph", &msg::MultiStageRuntime::graph, py::return_value_policy::reference_internal)
        .def_property_readonly("order", &msg::MultiStageRuntime::order)
        .def("set_factory", [](msg::MultiStageRuntime& rt, const std::string& runner, py::object factory) {
            auto held = std::shared_ptr<py::object>(new py::object(std::move(factory)), [](py::object* p) {
                py::gil_scoped_acquire gil;
                delete p;
            });
            rt.set_factory(runner, [held](const msg::StageSpec& spec, const std::string& root) {
                py::gil_scoped_acquire gil;
                return stage_fn_from_python((*held)(spec, root));
            });
        })
        .def("set_stage", [](msg::MultiStageRuntime& rt, const std::string& id, py::object fn) { rt.set_stage(id, stage_fn_from_python(std::move(fn))); })
        .def("stage_loaded", &msg::MultiStageRuntime::stage_loaded)
        .def("submit", [](msg::MultiStageRuntime& rt, const py::dict& fields, std::vector<std::string> want, const std::string& cohort_key,
                          std::shared_ptr<StreamChannel> text_sink, bool keep_unroutable) {
            msg::StageRequest r;
            r.fields = port_map_from_python(fields);
            r.want = std::move(want);
            r.cohort_key = cohort_key;
            r.text_sink = std::move(text_sink);
            std::string why;
            const int idx = rt.submit(std::move(r), &why, keep_unroutable);
            return py::make_tuple(idx, why);
        }, py::arg("fields"), py::arg("want") = std::vector<std::string>(), py::arg("cohort_key") = "", py::arg("text_sink") = nullptr,
           py::arg("keep_unroutable") = false)
        .def_property_readonly("pending", &msg::MultiStageRuntime::pending)
        .def("discard_pending", &msg::MultiStageRuntime::discard_pending)
        .def("cohorts", [](const msg::MultiStageRuntime& rt, int batch_size) {
            py::list out;
            for (auto& c : rt.cohorts(batch_size)) out.append(py::make_tuple(c.members, c.route));
            return out;
        }, py::arg("batch_size") = 1)
        .def("run", [](msg::MultiStageRuntime& rt, int batch_size) { return rt.run(batch_size); }, py::arg("batch_size") = 1)
        .def("take", &msg::MultiStageRuntime::take)
        .def("close", &msg::MultiStageRuntime::close)
        // one request, the way the reference's binding runs it: text always, audio terminals only when asked for
        .def("generate", [](msg::MultiStageRuntime& rt, const std::string& prompt, const std::string& style, const std::string& sampling, bool audio) {
            msg::StageRequest r;
            if (!prompt.empty()) r.fields["messages"] = msg::PortValue::text(prompt);
            if (!style.empty()) r.fields["style"] = msg::PortValue::text(style);
            if (!sampling.empty()) r.fields["sampling"] = msg::PortValue::text(sampling);
            for (const auto& t : rt.graph().terminals) {
                const size_t c = t.find(':');
                const msg::StageSpec& spec = rt.graph().stage(t.substr(0, c));
                for (const auto& e : spec.emits)
                    if (e.id == t.substr(c + 1) && (e.kind != "audio" || audio)) r.want.push_back(t);
            }
            MultiStageOutput out;
            r.audio_sink = [&out](const msg::PcmChunk& chunk) {
                out.audio_pcm16 += chunk.pcm16;
                out.audio_sample_rate = chunk.sample_rate;
                out.audio_channels = chunk.channels;
            };
            std::string why;
            if (rt.submit(std::move(r), &why) < 0) throw std::runtime_error("request refused: " + why);
            rt.run(1);
            const auto responses = rt.take();
            const msg::StageResponse& resp = responses.front();
            if (!resp.ok) throw std::runtime_error("request failed: " + resp.error);
            out.stages = resp.diagnostics().dump();
            for (const auto& kv : resp.outputs) {
                if (kv.second.kind == msg::PortValue::Kind::kText) out.text += kv.second.data;
                if (kv.second.kind == msg::PortValue::Kind::kTokens) out.token_ids = kv.second.tokens;
            }
            return out;
        }, py::arg("prompt"), py::arg("style") = "", py::arg("sampling") = "", py::arg("audio") = false);
}
