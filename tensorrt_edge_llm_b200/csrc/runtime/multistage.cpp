// Stage-graph runtime: config schema, validation, routes, cohorts and the run loop (see multistage.h).
#include "multistage.h"

#include <sys/stat.h>

#include <algorithm>
#include <chrono>
#include <fstream>
#include <sstream>

namespace telb {
namespace multistage {
namespace {

const char* const kOnMissing[] = {"fail", "skip", "prune"};

std::string join(const std::vector<std::string>& v, const char* sep = ", ") {
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) s += (i ? sep : "") + v[i];
    return s;
}

std::string quoted_list(std::vector<std::string> v) {
    std::sort(v.begin(), v.end());
    return "[" + join(v) + "]";
}

bool has(const std::vector<std::string>& v, const std::string& x) { return std::find(v.begin(), v.end(), x) != v.end(); }

const Json& required(const Json& obj, const char* key, size_t index) {
    const Json* p = obj.find(key);
    if (!p) throw GraphError("stages[" + std::to_string(index) + "] is missing '" + key + "'");
    return *p;
}

std::string stage_of(const std::string& terminal) { return terminal.substr(0, terminal.find(':')); }

}  // namespace

// ---- runner table ---------------------------------------------------------------------------------------------------

void RunnerTable::add(RunnerDecl d) {
    std::lock_guard<std::mutex> lk(mu_);
    decls_[d.name] = std::move(d);
}

bool RunnerTable::find(const std::string& name, RunnerDecl* out) const {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = decls_.find(name);
    if (it == decls_.end()) return false;
    if (out) *out = it->second;
    return true;
}

std::vector<std::string> RunnerTable::names() const {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<std::string> v;
    for (const auto& kv : decls_) v.push_back(kv.first);
    return v;
}

RunnerTable& RunnerTable::global() {
    static RunnerTable table;
    return table;
}

// ---- graph ------------------------------------------------------------------------------------------------------------

StageGraph StageGraph::parse(const Json& obj, const std::string& root) {
    if (!obj.is_object()) throw GraphError("the graph file must hold a JSON object");
    if (!obj["schema_version"].is_number() || obj["schema_version"].as_int() != kSchemaVersion)
        throw GraphError("schema_version must be " + std::to_string(kSchemaVersion));
    StageGraph g;
    g.root = root;
    size_t i = 0;
    for (const Json& s : obj["stages"].items()) {
        if (!s.is_object()) throw GraphError("stages[" + std::to_string(i) + "] must be an object");
        StageSpec spec;
        spec.id = required(s, "id", i).as_string();
        spec.runner = required(s, "runner", i).as_string();
        if (spec.id.empty() || spec.runner.empty()) throw GraphError("stages[" + std::to_string(i) + "] needs a non-empty id and runner");
        if (spec.id.find(':') != std::string::npos || spec.id == "request")
            throw GraphError("stages[" + std::to_string(i) + "]: the id may not contain ':' nor be 'request'");
        if (s.contains("artifact")) spec.artifact = s["artifact"].as_string();
        if (s.contains("kind")) spec.kind = s["kind"].as_string();
        for (const Json& p : s["inputs"].items()) {
            InputPort in;
            in.name = required(p, "name", i).as_string();
            in.source = required(p, "from", i).as_string();
            if (p.contains("on_missing")) in.on_missing = p["on_missing"].as_string();
            spec.inputs.push_back(std::move(in));
        }
        for (const Json& e : s["emits"].items()) {
            EmitPort out;
            out.id = required(e, "id", i).as_string();
            if (e.contains("kind")) out.kind = e["kind"].as_string();
            if (e.contains("transport")) out.transport = e["transport"].as_string();
            out.terminal = e["terminal"].as_bool(false);
            spec.emits.push_back(std::move(out));
        }
        spec.max_batch = static_cast<int>(s["max_batch"].as_int(0));
        spec.max_seq = static_cast<int>(s["max_seq"].as_int(0));
        if (s["config"].is_object()) spec.config = s["config"];
        g.stages.push_back(std::move(spec));
        ++i;
    }
    for (const Json& t : obj["terminals"].items()) g.terminals.push_back(t.as_string());
    return g;
}

StageGraph StageGraph::parse_text(const std::string& text, const std::string& root) {
    Json obj;
    try {
        obj = Json::parse(text);
    } catch (const std::exception& e) {
        throw GraphError(std::string("the graph file is not valid JSON: ") + e.what());
    }
    return parse(obj, root);
}

StageGraph StageGraph::load(const std::string& dir_or_file) {
    struct stat st {};
    std::string file = dir_or_file;
    if (::stat(dir_or_file.c_str(), &st) == 0 && S_ISDIR(st.st_mode)) file = dir_or_file + "/" + kConfigName;
    std::ifstream f(file, std::ios::binary);
    if (!f) throw GraphError("cannot open " + file);
    std::stringstream ss;
    ss << f.rdbuf();
    const size_t slash = file.find_last_of('/');
    return parse_text(ss.str(), slash == std::string::npos ? "." : file.substr(0, slash));
}

const StageSpec& StageGraph::stage(const std::string& id) const {
    for (const auto& s : stages)
        if (s.id == id) return s;
    throw GraphError("no stage named " + id);
}

std::vector<std::string> StageGraph::topological() const {
    std::map<std::string, std::set<std::string>> deps;
    for (const auto& s : stages) {
        auto& d = deps[s.id];
        for (const auto& p : s.inputs)
            if (!p.from_request()) d.insert(p.ref().first);
    }
    std::vector<std::string> order;
    std::set<std::string> done;
    while (!deps.empty()) {
        std::vector<std::string> ready;                  // std::map iterates in id order, which keeps the order stable
        for (const auto& kv : deps)
            if (std::all_of(kv.second.begin(), kv.second.end(), [&](const std::string& d) { return done.count(d) > 0; })) ready.push_back(kv.first);
        if (ready.empty()) {
            std::vector<std::string> left;
            for (const auto& kv : deps) left.push_back(kv.first);
            throw GraphError("the stages " + quoted_list(left) + " form a cycle");
        }
        for (const auto& r : ready) {
            order.push_back(r);
            deps.erase(r);
        }
        done.insert(ready.begin(), ready.end());
    }
    return order;
}

std::vector<std::string> StageGraph::validate(const RunnerTable* table) const {
    if (stages.empty()) throw GraphError("a graph needs at least one stage");
    std::set<std::string> ids;
    std::set<std::pair<std::string, std::string>> ports;
    for (const auto& s : stages) {
        if (!ids.insert(s.id).second) throw GraphError("stage ids must be unique (" + s.id + " appears twice)");
        for (const auto& e : s.emits)
            if (!ports.insert({s.id, e.id}).second) throw GraphError("stage " + s.id + ": duplicate output port " + e.id);
    }
    for (const auto& s : stages) {
        std::set<std::string> names;
        for (const auto& p : s.inputs) {
            if (!names.insert(p.name).second) throw GraphError("stage " + s.id + ": duplicate input " + p.name);
            if (std::find(std::begin(kOnMissing), std::end(kOnMissing), p.on_missing) == std::end(kOnMissing))
                throw GraphError("stage " + s.id + ": on_missing must be one of fail, skip, prune");
            if (p.source.find(':') == std::string::npos)
                throw GraphError("stage " + s.id + ": input '" + p.name + "' needs a source of the form <stage>:<port> or request:<field>");
            if (!p.from_request() && !ports.count(p.ref()))
                throw GraphError("stage " + s.id + ": input '" + p.name + "' reads '" + p.source + "', which no stage emits");
        }
        if (!table) continue;
        RunnerDecl decl;
        if (!table->find(s.runner, &decl))
            throw GraphError("stage " + s.id + ": unknown runner '" + s.runner + "'; known: " + quoted_list(table->names()));
        if (decl.kind != s.kind) throw GraphError("stage " + s.id + ": runner " + s.runner + " is " + decl.kind + ", the graph says " + s.kind);
        std::vector<std::string> bad_in, bad_out, bad_cfg;
        for (const auto& p : s.inputs)
            if (!decl.inputs.empty() && !has(decl.inputs, p.name)) bad_in.push_back(p.name);
        for (const auto& e : s.emits)
            if (!decl.emits.empty() && !has(decl.emits, e.id)) bad_out.push_back(e.id);
        for (const auto& k : decl.required_config)
            if (!s.config.contains(k)) bad_cfg.push_back(k);
        if (!bad_in.empty() || !bad_out.empty())
            throw GraphError("stage " + s.id + ": runner " + s.runner + " has no input " + quoted_list(bad_in) + " / output " + quoted_list(bad_out));
        if (!bad_cfg.empty()) throw GraphError("stage " + s.id + ": runner " + s.runner + " needs the config keys " + quoted_list(bad_cfg));
    }
    std::vector<std::string> marked;
    for (const auto& s : stages)
        for (const auto& e : s.emits)
            if (e.terminal) marked.push_back(s.id + ":" + e.id);
    for (const auto& t : terminals) {
        const size_t c = t.find(':');
        if (c == std::string::npos || !ports.count({t.substr(0, c), t.substr(c + 1)})) throw GraphError("terminal '" + t + "' is not an output of any stage");
    }
    std::vector<std::string> listed = terminals;
    std::sort(listed.begin(), listed.end());
    std::sort(marked.begin(), marked.end());
    if (listed != marked) throw GraphError("terminals " + quoted_list(listed) + " differ from the outputs marked terminal " + quoted_list(marked));
    return topological();
}

Json StageGraph::to_json() const {
    Json obj = Json::object();
    obj.set("schema_version", Json(kSchemaVersion));
    Json st = Json::array();
    for (const auto& s : stages) {
        Json e = Json::object();
        e.set("id", Json(s.id));
        e.set("runner", Json(s.runner));
        e.set("artifact", Json(s.artifact));
        e.set("kind", Json(s.kind));
        if (s.max_batch) e.set("max_batch", Json(s.max_batch));
        if (s.max_seq) e.set("max_seq", Json(s.max_seq));
        Json ins = Json::array();
        for (const auto& p : s.inputs) {
            Json j = Json::object();
            j.set("name", Json(p.name));
            j.set("from", Json(p.source));
            j.set("on_missing", Json(p.on_missing));
            ins.push_back(std::move(j));
        }
        e.set("inputs", std::move(ins));
        Json outs = Json::array();
        for (const auto& p : s.emits) {
            Json j = Json::object();
            j.set("id", Json(p.id));
            j.set("kind", Json(p.kind));
            j.set("transport", Json(p.transport));
            if (p.terminal) j.set("terminal", Json(true));
            outs.push_back(std::move(j));
        }
        e.set("emits", std::move(outs));
        if (s.config.size()) e.set("config", s.config);
        st.push_back(std::move(e));
    }
    obj.set("stages", std::move(st));
    Json term = Json::array();
    for (const auto& t : terminals) term.push_back(Json(t));
    obj.set("terminals", std::move(term));
    return obj;
}

// ---- routes -----------------------------------------------------------------------------------------------------------

Route plan_route(const StageGraph& g, const std::set<std::string>& fields, const std::vector<std::string>* want_in) {
    const std::vector<std::string> order = g.topological();
    const std::vector<std::string>& want = want_in ? *want_in : g.terminals;
    Route r;
    std::set<std::string> runnable;
    for (const auto& sid : order) {
        const StageSpec& s = g.stage(sid);
        std::string why;
        for (const auto& p : s.inputs) {
            const bool present = p.from_request() ? fields.count(p.ref().second) > 0 : runnable.count(p.ref().first) > 0;
            if (!present && p.on_missing != "skip") {
                why = "input '" + p.name + "' (" + p.source + ") is missing";
                break;
            }
        }
        if (why.empty()) runnable.insert(sid);
        else r.skipped.emplace_back(sid, why);
    }
    // of the stages that can run, keep those that feed a requested terminal
    std::set<std::string> needed;
    std::vector<std::string> frontier;
    for (const auto& t : want) frontier.push_back(stage_of(t));
    while (!frontier.empty()) {
        const std::string sid = frontier.back();
        frontier.pop_back();
        if (needed.count(sid) || !runnable.count(sid)) continue;
        needed.insert(sid);
        for (const auto& p : g.stage(sid).inputs)
            if (!p.from_request() && runnable.count(p.ref().first)) frontier.push_back(p.ref().first);
    }
    std::vector<std::string> missing;
    for (const auto& t : want) (needed.count(stage_of(t)) ? r.terminals : missing).push_back(t);
    for (const auto& sid : order)
        if (needed.count(sid)) r.stages.push_back(sid);
    for (size_t i = 0; i < missing.size(); ++i) {
        const std::string sid = stage_of(missing[i]);
        const std::string* why = r.why_skipped(sid);
        r.error += (i ? "; " : "") + missing[i] + " needs stage " + sid + ": " + (why ? *why : std::string("an upstream stage cannot run"));
    }
    return r;
}

// ---- responses --------------------------------------------------------------------------------------------------------

Json StageResponse::diagnostics() const {
    Json obj = Json::object();
    for (const auto& kv : stages) {
        Json d = Json::object();
        d.set("ran", Json(kv.second.ran));
        if (kv.second.ran) {
            d.set("batch", Json(kv.second.batch));
            d.set("seconds", Json(kv.second.seconds));
        } else {
            d.set("reason", Json(kv.second.reason));
        }
        obj.set(kv.first, std::move(d));
    }
    return obj;
}

// ---- runtime ----------------------------------------------------------------------------------------------------------

void MultiStageRuntime::load(StageGraph g, bool check_runners) {
    order_ = g.validate(check_runners ? &RunnerTable::global() : nullptr);
    graph_ = std::move(g);
    loaded_.clear();
    pending_.clear();
    responses_.clear();
}

void MultiStageRuntime::set_factory(const std::string& runner, StageFactory f) { factories_[runner] = std::move(f); }

void MultiStageRuntime::set_stage(const std::string& stage_id, StageFn fn) {
    graph_.stage(stage_id);                               // throws for an id the graph does not have
    loaded_[stage_id] = std::move(fn);
}

bool MultiStageRuntime::stage_loaded(const std::string& stage_id) const { return loaded_.count(stage_id) > 0; }

StageFn& MultiStageRuntime::stage_fn(const std::string& id) {
    auto it = loaded_.find(id);
    if (it != loaded_.end()) return it->second;
    // stages load on first use: a text-only run never loads the vocoder
    const StageSpec& spec = graph_.stage(id);
    auto f = factories_.find(spec.runner);
    if (f == factories_.end()) throw GraphError("stage " + id + ": no factory for runner '" + spec.runner + "'");
    return loaded_[id] = f->second(spec, graph_.root);
}

int MultiStageRuntime::submit(StageRequest r, std::string* error, bool keep_unroutable) {
    std::set<std::string> fields;
    for (const auto& kv : r.fields)
        if (kv.second.present()) fields.insert(kv.first);
    for (const auto& t : r.want)
        if (!has(graph_.terminals, t)) {
            if (error) *error = "'" + t + "' is not a terminal of this graph; terminals: " + quoted_list(graph_.terminals);
            return -1;
        }
    const Route route = plan_route(graph_, fields, r.want.empty() ? nullptr : &r.want);
    if (route.terminals.empty() && !keep_unroutable) {
        if (error) *error = route.error.empty() ? "the request reaches no terminal" : route.error;
        return -1;
    }
    pending_.push_back(std::move(r));
    return static_cast<int>(pending_.size()) - 1;
}

std::vector<MultiStageRuntime::Cohort> MultiStageRuntime::cohorts(int batch_size) const {
    int cap = std::max(batch_size, 1);
    for (const auto& s : graph_.stages)
        if (s.max_batch) cap = std::min(cap, s.max_batch);
    cap = std::max(cap, 1);
    std::vector<Cohort> out;
    std::vector<std::string> keys;
    for (size_t i = 0; i < pending_.size(); ++i) {
        const StageRequest& r = pending_[i];
        std::set<std::string> fields;
        for (const auto& kv : r.fields)
            if (kv.second.present()) fields.insert(kv.first);
        Route route = plan_route(graph_, fields, r.want.empty() ? nullptr : &r.want);
        const std::string key = join(route.stages, ">") + "|" + join(route.terminals, ",") + "|" + r.cohort_key;
        bool placed = false;
        for (size_t c = 0; c < out.size() && !placed; ++c)
            if (keys[c] == key && static_cast<int>(out[c].members.size()) < cap) {
                out[c].members.push_back(static_cast<int>(i));
                placed = true;
            }
        if (!placed) {
            keys.push_back(key);
            out.push_back(Cohort{{static_cast<int>(i)}, std::move(route)});
        }
    }
    return out;
}

const std::vector<StageResponse>& MultiStageRuntime::run(int batch_size) {
    responses_.assign(pending_.size(), StageResponse());
    for (const Cohort& cohort : cohorts(batch_size)) {
        const size_t nreq = cohort.members.size();
        std::vector<std::map<std::pair<std::string, std::string>, PortValue>> values(nreq);
        std::vector<std::pair<std::string, StageDiag>> detail;
        for (const auto& kv : cohort.route.skipped) {
            StageDiag d;
            d.reason = kv.second;
            detail.emplace_back(kv.first, std::move(d));
        }
        std::string error = cohort.route.error;
        for (const auto& sid : cohort.route.stages) {
            const StageSpec& spec = graph_.stage(sid);
            std::vector<PortMap> batch(nreq);
            for (size_t j = 0; j < nreq; ++j)
                for (const auto& p : spec.inputs) {
                    const PortValue* src = nullptr;
                    if (p.from_request()) {
                        auto it = pending_[cohort.members[j]].fields.find(p.ref().second);
                        if (it != pending_[cohort.members[j]].fields.end()) src = &it->second;
                    } else {
                        auto it = values[j].find(p.ref());
                        if (it != values[j].end()) src = &it->second;
                    }
                    if (src && src->present()) batch[j][p.name] = *src;
                }
            StageDiag d;
            const auto t0 = std::chrono::steady_clock::now();
            try {
                RunnerDecl decl;
                const bool one_by_one = RunnerTable::global().find(spec.runner, &decl) && !decl.batches && nreq > 1;
                StageFn& fn = stage_fn(sid);
                std::vector<PortMap> outs;
                if (one_by_one) {
                    for (size_t j = 0; j < nreq; ++j) {
                        std::vector<PortMap> one = fn(spec, std::vector<PortMap>{batch[j]});
                        if (one.size() != 1) throw GraphError("the stage returned " + std::to_string(one.size()) + " results for one request");
                        outs.push_back(std::move(one[0]));
                    }
                } else {
                    outs = fn(spec, batch);
                }
                if (outs.size() != nreq)
                    throw GraphError("the stage returned " + std::to_string(outs.size()) + " results for " + std::to_string(nreq) + " requests");
                for (size_t j = 0; j < nreq; ++j)
                    for (auto& kv : outs[j]) values[j][{sid, kv.first}] = std::move(kv.second);
                d.ran = true;
                d.batch = static_cast<int>(nreq);
            } catch (const std::exception& e) {
                error = "stage " + sid + ": " + e.what();
                d.reason = error;
            }
            d.seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            const bool failed = !d.ran;
            detail.emplace_back(sid, std::move(d));
            if (failed) break;
        }
        for (size_t j = 0; j < nreq; ++j) {
            const StageRequest& req = pending_[cohort.members[j]];
            StageResponse& resp = responses_[cohort.members[j]];
            bool all = true;
            for (const auto& t : cohort.route.terminals) {
                const size_t c = t.find(':');
                auto it = values[j].find({t.substr(0, c), t.substr(c + 1)});
                PortValue v = it == values[j].end() ? PortValue() : it->second;
                all = all && v.present();
                resp.outputs.emplace_back(t, std::move(v));
            }
            resp.ok = error.empty() && all;
            if (!resp.ok) resp.error = error.empty() ? "a terminal produced nothing" : error;
            resp.stages = detail;
            // sinks: text terminals as one finished chunk, audio terminals that carry bytes as one PCM chunk
            for (const auto& kv : resp.outputs) {
                const size_t c = kv.first.find(':');
                const StageSpec& spec = graph_.stage(kv.first.substr(0, c));
                const auto port = std::find_if(spec.emits.begin(), spec.emits.end(), [&](const EmitPort& e) { return e.id == kv.first.substr(c + 1); });
                if (port == spec.emits.end()) continue;
                if (port->kind == "audio" && req.audio_sink && kv.second.kind == PortValue::Kind::kBytes) {
                    PcmChunk chunk;
                    chunk.pcm16 = kv.second.data;
                    chunk.sample_rate = static_cast<int>(spec.config["sample_rate"].as_int(24000));
                    chunk.channels = static_cast<int>(spec.config["channels"].as_int(1));
                    req.audio_sink(chunk);
                }
            }
            if (req.text_sink) {
                for (const auto& kv : resp.outputs)
                    if (kv.second.kind == PortValue::Kind::kTokens) req.text_sink->push(kv.second.tokens);
                req.text_sink->finish(resp.ok ? FinishReason::kEndId : FinishReason::kError);
            }
        }
    }
    pending_.clear();
    return responses_;
}

std::vector<StageResponse> MultiStageRuntime::take() {
    std::vector<StageResponse> out;
    out.swap(responses_);
    return out;
}

void MultiStageRuntime::close() {
    loaded_.clear();
    pending_.clear();
    responses_.clear();
}

}  // namespace multistage
}  // namespace telb
