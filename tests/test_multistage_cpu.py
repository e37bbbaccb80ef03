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
    assert ("thinker", 2) in Scripted.calls and res[0]["stages"]["talker"] == {"ran": True, "batch": 2}
    text_only = rt.run(reqs[:1], want=["thinker:text"])
    assert text_only[0]["outputs"] == {"thinker:text": "re:ab"} and "talker" not in text_only[0]["stages"]


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
