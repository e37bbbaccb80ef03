"""Stage graph: parsing, validation, per-request routing, cohorts, execution with scripted stages and the LLM backbone."""
import json
import os

import pytest

from tensorrt_edge_llm_b200.runtime import multistage as ms


class Scripted(ms.Stage):
    calls = []

    def run(self, batch):
        Scripted.calls.append((self.cfg.id, len(batch)))
        fn = {"thinker": lambda r: {"text": "re:" + r["prompt"], "accept_hidden": [len(r["prompt"])]},
              "talker": lambda r: {"codes": [ord(c) for c in r["text_ids"]] + ([7] if r.get("voice") else [])},
              "code2wav": lambda r: {"audio": [c * 2 for c in r["codes"]]}}[self.cfg.id]
        return [fn(r) for r in batch]


for name, kind in (("test.thinker", "autoregressive"), ("test.talker", "autoregressive"), ("test.code2wav", "iterative")):
    ms.register_runner(ms.RunnerDecl(name, kind, Scripted))

OMNI = {"schema_version": 1, "terminals": ["thinker:text", "code2wav:audio"], "stages": [
    {"id": "code2wav", "runner": "test.code2wav", "artifact": "code2wav", "kind": "iterative",
     "inputs": [{"name": "codes", "from": "talker:codes"}], "emits": [{"id": "audio", "kind": "audio", "terminal": True}]},
    {"id": "thinker", "runner": "test.thinker", "kind": "autoregressive", "max_batch": 2,
     "inputs": [{"name": "prompt", "from": "request:messages"}, {"name": "audio", "from": "request:audio", "on_missing": "skip"}],
     "emits": [{"id": "text", "kind": "text", "terminal": True}, {"id": "accept_hidden", "kind": "hidden"}]},
    {"id": "talker", "runner": "test.talker", "artifact": "talker", "kind": "autoregressive",
     "inputs": [{"name": "hidden", "from": "thinker:accept_hidden"}, {"name": "text_ids", "from": "thinker:text"},
                {"name": "voice", "from": "request:voice", "on_missing": "skip"}],
     "emits": [{"id": "codes", "kind": "codec"}]}]}


def test_parse_validate_and_order():
    g = ms.parse_graph(OMNI)
    assert ms.validate_graph(g) == ["thinker", "talker", "code2wav"]
    for mutate, msg in [
        (lambda o: o.update(schema_version=3), "schema_version"),
        (lambda o: o["stages"][0].update(runner="nope"), "unknown runner"),
        (lambda o: o["stages"][0].update(kind="autoregressive"), "is iterative"),
        (lambda o: o["stages"][0]["inputs"][0].update({"from": "talker:nothing"}), "no stage emits"),
        (lambda o: o["stages"][1]["inputs"][0].update(on_missing="maybe"), "on_missing"),
        (lambda o: o.update(terminals=["thinker:text"]), "differ from"),
        (lambda o: o["stages"][1]["inputs"].append({"name": "loop", "from": "code2wav:audio"}), "cycle"),
        (lambda o: o["stages"].append(dict(o["stages"][0])), "unique"),
    ]:
        bad = json.loads(json.dumps(OMNI))
        mutate(bad)
        with pytest.raises(ms.GraphConfigError, match=msg):
            ms.parse_graph(bad)


def test_routing_prunes_to_requested_terminals():
    g = ms.parse_graph(OMNI)
    r = ms.plan_route(g, {"messages": "hi"}, ["thinker:text"])
    assert r.stages == ["thinker"] and r.error is None                    # text only: the speech stages do not run
    r = ms.plan_route(g, {"messages": "hi"})
    assert r.stages == ["thinker", "talker", "code2wav"] and r.terminals == ["thinker:text", "code2wav:audio"]
    r = ms.plan_route(g, {"audio": b"x"})                                  # no prompt: nothing can run
    assert r.stages == [] and "messages" in r.error and set(r.skipped) == {"thinker", "talker", "code2wav"}


def test_cohorts_and_execution():
    Scripted.calls = []
    rt = ms.MultiStageRuntime(ms.parse_graph(OMNI))
    reqs = [{"messages": "ab"}, {"messages": "c", "voice": "v1"}, {"messages": "de"}, {"messages": "f"}, {"audio": 1}]
    cohorts = rt.cohorts(reqs, None, batch_size=4)
    assert [idx for idx, _ in cohorts] == [[0, 2], [1], [3], [4]]         # thinker's max_batch 2 caps the cohort; a voice splits it
    res = rt.run(reqs, batch_size=4)
    assert res[0]["ok"] and res[0]["outputs"] == {"thinker:text": "re:ab", "code2wav:audio": [2 * ord(c) for c in "re:ab"]}
    assert res[1]["outputs"]["code2wav:audio"][-1] == 14 and res[2]["outputs"]["thinker:text"] == "re:de"
    assert not res[4]["ok"] and "missing" in res[4]["error"]
    assert ("thinker", 2) in Scripted.calls and {k: res[0]["stages"]["talker"][k] for k in ("ran", "batch")} == {"ran": True, "batch": 2}
    text_only = rt.run(reqs[:1], want=["thinker:text"])
    assert text_only[0]["outputs"] == {"thinker:text": "re:ab"} and "talker" not in text_only[0]["stages"]


def test_native_runtime_surface(tmp_path):
    """The native class itself: load from a directory, stages as callables or through a factory, refusal at submit,
    ``generate`` for one request, a runner that does not batch, a failing stage, token terminals on a stream channel."""
    from tensorrt_edge_llm_b200.runtime import native as rt
    nms = rt.multistage
    nms.register_runner("native.echo", "autoregressive", ["prompt", "style"], ["text", "ids"], [], False)
    nms.register_runner("native.voice", "iterative", ["text"], ["audio"], ["sample_rate"])
    graph = {"schema_version": 1, "terminals": ["echo:text", "echo:ids", "voice:audio"], "stages": [
        {"id": "echo", "runner": "native.echo", "kind": "autoregressive",
         "inputs": [{"name": "prompt", "from": "request:messages"}, {"name": "style", "from": "request:style", "on_missing": "skip"}],
         "emits": [{"id": "text", "kind": "text", "terminal": True}, {"id": "ids", "kind": "tokens", "terminal": True}]},
        {"id": "voice", "runner": "native.voice", "kind": "iterative", "config": {"sample_rate": 16000},
         "inputs": [{"name": "text", "from": "echo:text"}], "emits": [{"id": "audio", "kind": "audio", "terminal": True}]}]}
    (tmp_path / nms.CONFIG_NAME).write_text(json.dumps(graph))
    m = nms.MultiStageRuntime(str(tmp_path))
    assert m.order == ["echo", "voice"] and m.graph.root == str(tmp_path) and json.loads(m.graph.to_json())["terminals"] == graph["terminals"]
    sizes = []

    def echo(spec, batch):
        sizes.append(len(batch))
        return [{"text": (r.get("style", "") + r["prompt"]).upper(), "ids": [len(r["prompt"]), 7]} for r in batch]

    built = []

    def voice_factory(spec, root):
        built.append((spec.id, root, json.loads(spec.config_json)["sample_rate"]))
        return lambda spec, batch: [{"audio": r["text"].encode() * 2} for r in batch]

    m.set_stage("echo", echo)
    m.set_factory("native.voice", voice_factory)
    out = m.generate("hi", style="x")                               # text only: the voice stage is neither built nor run
    assert out.text == "XHI" and built == [] and not m.stage_loaded("voice") and "voice" not in json.loads(out.stages)
    out = m.generate("hi", audio=True)
    assert out.audio_pcm16 == b"HIHI" and out.audio_sample_rate == 16000 and built == [("voice", str(tmp_path), 16000)]
    with pytest.raises(RuntimeError, match="refused.*messages"):
        m.generate("")                                              # no prompt: no terminal can be produced
    assert m.submit({"messages": "a"}, ["echo:nothing"])[0] == -1
    # a runner declared as not batching sees the cohort one request at a time
    sizes.clear()
    chan = rt.StreamChannel.create()
    for i, text in enumerate(("a", "bb", "ccc")):
        assert m.submit({"messages": text}, ["echo:ids"], "", chan if i == 0 else None)[0] == i
    assert [members for members, _ in m.cohorts(8)] == [[0, 1, 2]]
    res = m.run(8)
    assert sizes == [1, 1, 1] and [r.outputs["echo:ids"] for r in res] == [[1, 7], [2, 7], [3, 7]] and m.pending == 0
    chunk = chan.try_pop()
    assert list(chunk.token_ids) == [1, 7] and chan.is_finished()
    # a stage that raises fails its cohort with the stage named; a later run is unaffected
    m.set_stage("echo", lambda spec, batch: (_ for _ in ()).throw(ValueError("boom")))
    m.submit({"messages": "a"}, ["echo:text"])
    r = m.run()[0]
    assert not r.ok and "stage echo" in r.error and "boom" in r.error
    # required config keys are part of the runner's declaration
    del graph["stages"][1]["config"]
    with pytest.raises(nms.GraphError, match="sample_rate"):
        nms.StageGraph.parse_text(json.dumps(graph)).validate()


def test_one_stage_graph_with_the_llm_backbone(tmp_path):
    from tensorrt_edge_llm_b200.cli import main as trtedge
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    d = str(tmp_path)
    assert trtedge(["multistage", "--config", d, "--write-one-stage-graph"]) == 0
    assert trtedge(["multistage", "--config", d, "--validate-config"]) == 0
    g = ms.load_graph(d)
    llm = LLM(tiny_llama_config(num_hidden_layers=1), device="cpu", max_batch_size=2, max_input_len=32, max_kv_cache_capacity=64, page_size=16)
    rt = ms.MultiStageRuntime(g, stages={"llm": ms.LLMBackboneStage(g.stage("llm"), d, llm=llm)})
    res = rt.run([{"messages": [3, 4, 5], "sampling": {"max_tokens": 4}}, {"messages": [6, 7], "sampling": {"max_tokens": 4}}], batch_size=2)
    assert all(r["ok"] for r in res) and res[0]["stages"]["llm"]["batch"] == 2
    want = llm.generate([[3, 4, 5]], __import__("tensorrt_edge_llm_b200.runtime.llm", fromlist=["SamplingParams"]).SamplingParams(max_tokens=4))
    rt2 = ms.MultiStageRuntime(g, stages={"llm": ms.LLMBackboneStage(g.stage("llm"), d, llm=llm)})
    got = rt2.run([{"messages": [3, 4, 5], "sampling": {"max_tokens": 4}}], want=["llm:text"])
    assert got[0]["ok"] and want[0].token_ids is not None
    open(os.path.join(d, "multistage_config.json"), "w").write("{}")
    assert trtedge(["multistage", "--config", d, "--validate-config"]) == 1
