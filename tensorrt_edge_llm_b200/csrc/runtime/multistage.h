// Stage-graph runtime: a deployment is a JSON list of stages (text decoder, encoders, talker, vocoder …) and of the
// edges between their ports; the runtime knows no model family.  A request runs only the stages whose inputs it can
// supply and whose outputs reach a terminal it asked for; requests that run the same stages with the same batch-wide
// settings form a cohort and go through each stage as one batch.
//
// Counterpart of cpp/runtime/multiStage/ in the reference (multiStageRuntime.{h,cpp}: load / submit / run / take;
// stageConfig.{h,cpp}: the multistage_config.json schema and validate(); route.{h,cpp}: per-request routes and
// on_missing; stageRegistry.{h,cpp}: the runner table with declarations; sinks.cpp: text / audio sinks) and of the
// guide docs/source/developer_guide/software-design/multi-stage-graph.md.
#pragma once

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "json.h"
#include "streaming.h"

namespace telb {
namespace multistage {

constexpr int kSchemaVersion = 1;
constexpr const char* kConfigName = "multistage_config.json";

class GraphError : public std::runtime_error {
  public:
    using std::runtime_error::runtime_error;
};

struct InputPort {
    std::string name;
    std::string source;                     // "request:<field>" or "<stage>:<port>"
    std::string on_missing = "fail";        // fail | skip | prune
    bool from_request() const { return source.compare(0, 8, "request:") == 0; }
    std::pair<std::string, std::string> ref() const {
        const size_t c = source.find(':');
        return c == std::string::npos ? std::make_pair(source, std::string()) : std::make_pair(source.substr(0, c), source.substr(c + 1));
    }
};

struct EmitPort {
    std::string id;
    std::string kind = "tensor";
    std::string transport = "chunk_stream";
    bool terminal = false;
};

struct StageSpec {
    std::string id, runner, artifact = ".", kind = "autoregressive";
    std::vector<InputPort> inputs;
    std::vector<EmitPort> emits;
    int max_batch = 0, max_seq = 0;
    Json config = Json::object();
};

// What a runner accepts and produces; an empty list means "anything".
struct RunnerDecl {
    std::string name, kind;
    std::vector<std::string> inputs, emits;
    std::vector<std::string> required_config;   // keys the stage entry's "config" object must carry
    bool batches = true;                        // false: the stage takes one request at a time whatever the cohort size
};

class RunnerTable {
  public:
    void add(RunnerDecl d);
    bool find(const std::string& name, RunnerDecl* out) const;
    std::vector<std::string> names() const;
    static RunnerTable& global();

  private:
    mutable std::mutex mu_;
    std::map<std::string, RunnerDecl> decls_;
};

struct StageGraph {
    std::vector<StageSpec> stages;
    std::vector<std::string> terminals;
    std::string root = ".";

    static StageGraph parse(const Json& obj, const std::string& root = ".");
    static StageGraph parse_text(const std::string& text, const std::string& root = ".");
    static StageGraph load(const std::string& dir_or_file);       // <dir>/multistage_config.json, or the file itself
    const StageSpec& stage(const std::string& id) const;
    // Structure checks and, with a table, agreement of every stage with its runner's declaration.  Returns the
    // execution order.  Throws GraphError with the first finding.
    std::vector<std::string> validate(const RunnerTable* table) const;
    std::vector<std::string> topological() const;
    Json to_json() const;
};

struct Route {
    std::vector<std::string> stages;                              // in execution order
    std::vector<std::string> terminals;                           // the requested terminals the request will receive
    std::vector<std::pair<std::string, std::string>> skipped;     // stage id → why it cannot run
    std::string error;                                            // non-empty when a requested terminal is out of reach
    const std::string* why_skipped(const std::string& id) const {
        for (const auto& kv : skipped)
            if (kv.first == id) return &kv.second;
        return nullptr;
    }
};

// `fields`: the request fields that are present.  `want`: null = every terminal of the graph.
Route plan_route(const StageGraph& g, const std::set<std::string>& fields, const std::vector<std::string>* want);

// A value on an edge.  Text and bytes travel as such; token ids and float tensors have typed forms for native stages;
// anything else (a device tensor owned by a binding, a host object) rides in `opaque`.
struct PortValue {
    enum class Kind { kNone, kText, kBytes, kTokens, kFloats, kOpaque };
    Kind kind = Kind::kNone;
    std::string data;                       // kText / kBytes
    std::vector<int32_t> tokens;            // kTokens
    std::vector<float> values;              // kFloats
    std::vector<int64_t> shape;             // kFloats
    std::shared_ptr<void> opaque;           // kOpaque
    bool present() const { return kind != Kind::kNone; }
    static PortValue text(std::string s) { PortValue v; v.kind = Kind::kText; v.data = std::move(s); return v; }
    static PortValue bytes(std::string s) { PortValue v; v.kind = Kind::kBytes; v.data = std::move(s); return v; }
    static PortValue token_ids(std::vector<int32_t> t) { PortValue v; v.kind = Kind::kTokens; v.tokens = std::move(t); return v; }
    static PortValue floats(std::vector<float> f, std::vector<int64_t> shape) {
        PortValue v; v.kind = Kind::kFloats; v.values = std::move(f); v.shape = std::move(shape); return v;
    }
    static PortValue object(std::shared_ptr<void> p) { PortValue v; v.kind = Kind::kOpaque; v.opaque = std::move(p); return v; }
};
using PortMap = std::map<std::string, PortValue>;

struct PcmChunk {
    std::string pcm16;                      // little-endian 16-bit samples
    int sample_rate = 0, channels = 1;
};

struct StageRequest {
    PortMap fields;                                   // request:<field> values
    std::vector<std::string> want;                    // empty = every terminal
    std::string cohort_key;                           // requests share a cohort only when this agrees (sampling, voice …)
    std::shared_ptr<StreamChannel> text_sink;         // optional: terminals that carry token ids are also pushed here, then the channel is finished
    std::function<void(const PcmChunk&)> audio_sink;  // optional: terminals of kind "audio" carrying bytes
};

struct StageDiag {
    bool ran = false;
    int batch = 0;
    double seconds = 0.0;
    std::string reason;
};

struct StageResponse {
    bool ok = false;
    std::string error;
    std::vector<std::pair<std::string, PortValue>> outputs;       // terminal id → value, in the order requested
    std::vector<std::pair<std::string, StageDiag>> stages;
    Json diagnostics() const;
    const PortValue* output(const std::string& terminal) const {
        for (const auto& kv : outputs)
            if (kv.first == terminal) return &kv.second;
        return nullptr;
    }
};

// One loaded stage: per request of the cohort, its resolved inputs in; per request, port id → value out.
using StageFn = std::function<std::vector<PortMap>(const StageSpec&, const std::vector<PortMap>&)>;
// Builds a stage from its graph entry and the graph's root directory (called on first use of the stage).
using StageFactory = std::function<StageFn(const StageSpec&, const std::string& root)>;

class MultiStageRuntime {
  public:
    struct Cohort {
        std::vector<int> members;           // indices into the pending list
        Route route;
    };

    // `check_runners`: validate every stage against RunnerTable::global() (off when stages are handed in directly).
    void load(StageGraph g, bool check_runners = true);
    void load_dir(const std::string& dir_or_file, bool check_runners = true) { load(StageGraph::load(dir_or_file), check_runners); }
    const StageGraph& graph() const { return graph_; }
    const std::vector<std::string>& order() const { return order_; }

    void set_factory(const std::string& runner, StageFactory f);
    void set_stage(const std::string& stage_id, StageFn fn);
    bool stage_loaded(const std::string& stage_id) const;

    // Queues a request.  Returns its index in the next run(), or -1 with `error` set when no requested terminal can be
    // produced for it (the request is refused, nothing is queued).  With `keep_unroutable` such a request is queued all
    // the same and run() answers it with a failed response that carries the route's explanation.
    int submit(StageRequest r, std::string* error = nullptr, bool keep_unroutable = false);
    size_t pending() const { return pending_.size(); }
    void discard_pending() { pending_.clear(); }
    std::vector<Cohort> cohorts(int batch_size) const;
    // Runs everything queued, cohort by cohort; a failing stage fails its cohort, not the run.  Responses are in
    // submission order and stay available through take() until the next run().
    const std::vector<StageResponse>& run(int batch_size = 1);
    std::vector<StageResponse> take();
    void close();

  private:
    StageFn& stage_fn(const std::string& id);
    StageGraph graph_;
    std::vector<std::string> order_;
    std::map<std::string, StageFactory> factories_;
    std::map<std::string, StageFn> loaded_;
    std::vector<StageRequest> pending_;
    std::vector<StageResponse> responses_;
};

}  // namespace multistage
}  // namespace telb
