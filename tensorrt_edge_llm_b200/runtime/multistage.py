"""Multi-stage runtime: a JSON-described graph of stages (LLM backbone, encoders, talker, vocoder …) run per cohort.

Follows ``cpp/runtime/multiStage/`` (``multiStageRuntime``, ``route``, ``stageConfig``, stage registry and factories)
and ``docs/source/developer_guide/software-design/multi-stage-graph.md``: ``multistage_config.json`` lists stages
(``id``, ``runner``, ``artifact``, ``kind``, ``inputs[{name, from, on_missing}]``, ``emits[{id, kind, transport,
terminal}]``) and ``terminals``; a request runs only the stages whose inputs it can supply and whose outputs reach a
requested terminal; requests that run the same stages form a cohort of at most ``max_batch``.

The schema, its validation, the routes, the cohorts and the run loop are the native runtime's
(``csrc/runtime/multistage.{h,cpp}``, bound as ``runtime.native.multistage``); this module is the Python face of it:
dataclass views of a parsed graph, the table of Python stage classes, and a ``MultiStageRuntime`` that plugs those
classes into the native loop as callables.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

from . import native as _rt

_ms = _rt.multistage
SCHEMA_VERSION = _ms.SCHEMA_VERSION
CONFIG_NAME = _ms.CONFIG_NAME
GraphConfigError = _ms.GraphError                      # a ValueError


@dataclass
class InputPort:
    name: str
    source: str                       # "request:<field>" or "<stage>:<port>"
    on_missing: str = "fail"

    @property
    def from_request(self) -> bool:
        return self.source.startswith("request:")

    @property
    def ref(self) -> Tuple[str, str]:
        a, _, b = self.source.partition(":")
        return a, b


@dataclass
class EmitPort:
    id: str
    kind: str
    transport: str = "chunk_stream"
    terminal: bool = False


@dataclass
class StageConfig:
    id: str
    runner: str
    artifact: str = "."
    kind: str = "autoregressive"
    inputs: List[InputPort] = field(default_factory=list)
    emits: List[EmitPort] = field(default_factory=list)
    max_batch: int = 0
    max_seq: int = 0
    config: Dict[str, Any] = field(default_factory=dict)


@dataclass
class GraphConfig:
    stages: List[StageConfig]
    terminals: List[str]
    root: str = "."
    native: Any = None                    # the parsed native graph these views were made from

    def stage(self, sid: str) -> StageConfig:
        for s in self.stages:
            if s.id == sid:
                return s
        raise KeyError(sid)

    def to_dict(self) -> Dict[str, Any]:
        return {"schema_version": SCHEMA_VERSION, "terminals": list(self.terminals), "stages": [
            {"id": s.id, "runner": s.runner, "artifact": s.artifact, "kind": s.kind, "max_batch": s.max_batch, "max_seq": s.max_seq,
             "config": s.config, "inputs": [{"name": p.name, "from": p.source, "on_missing": p.on_missing} for p in s.inputs],
             "emits": [{"id": e.id, "kind": e.kind, "transport": e.transport, "terminal": e.terminal} for e in s.emits]}
            for s in self.stages]}


def _native_graph(g: GraphConfig):
    if g.native is None:                  # a graph assembled from the dataclasses by hand
        g.native = _ms.StageGraph.parse_text(json.dumps(g.to_dict()), g.root)
    return g.native


def _view(ng) -> GraphConfig:
    stages = [StageConfig(s.id, s.runner, s.artifact, s.kind, [InputPort(p.name, p.source, p.on_missing) for p in s.inputs],
                          [EmitPort(e.id, e.kind, e.transport, e.terminal) for e in s.emits], s.max_batch, s.max_seq, json.loads(s.config_json))
              for s in ng.stages]
    return GraphConfig(stages, list(ng.terminals), ng.root, ng)


# ---- runner table ----------------------------------------------------------------------------------------------------

@dataclass
class RunnerDecl:
    name: str
    kind: str
    factory: Callable[[StageConfig, str], "Stage"]
    inputs: Tuple[str, ...] = ()          # input names the runner understands (empty = any)
    emits: Tuple[str, ...] = ()           # ports it can produce (empty = any)


class Stage:
    """One loaded stage.  ``run(batch)`` receives, per request of the cohort, a dict of its resolved inputs and
    returns, per request, a dict port id → value."""

    def __init__(self, cfg: StageConfig, root: str):
        self.cfg, self.root = cfg, root

    def run(self, batch: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        raise NotImplementedError

    def close(self) -> None:
        pass


_RUNNERS: Dict[str, RunnerDecl] = {}


def register_runner(decl: RunnerDecl) -> None:
    _RUNNERS[decl.name] = decl
    _ms.register_runner(decl.name, decl.kind, list(decl.inputs), list(decl.emits))


def runner_names() -> List[str]:
    return sorted(_RUNNERS)


class LLMBackboneStage(Stage):
    """``llm.backbone``: the text decoder of the artifact directory behind the ordinary ``LLM`` front end."""

    def __init__(self, cfg: StageConfig, root: str, llm=None):
        super().__init__(cfg, root)
        if llm is None:
            from .llm import LLM
            llm = LLM(os.path.normpath(os.path.join(root, cfg.artifact)), max_batch_size=cfg.max_batch or 8,
                      **{k: v for k, v in cfg.config.items() if k in ("max_input_len", "max_kv_cache_capacity", "device", "page_size")})
        self.llm = llm

    def run(self, batch):
        from .runner import SamplingParams
        prompts = []
        for r in batch:
            p = r.get("prompt")
            if isinstance(p, list) and p and isinstance(p[0], dict):          # chat messages
                from ..chat_template import ChatTemplate
                p = ChatTemplate().apply(p, True)
            prompts.append(p)
        s0 = batch[0].get("sampling") or {}
        sp = SamplingParams(max_tokens=int(s0.get("max_tokens", self.cfg.config.get("max_tokens", 64))),
                            temperature=float(s0.get("temperature", 0.0)), top_k=int(s0.get("top_k", 0)), top_p=float(s0.get("top_p", 1.0)),
                            seed=int(s0.get("seed", 42)))
        outs = self.llm.generate(prompts, sp)
        return [{"text": o.text if o.text is not None else "", "token_ids": o.token_ids, "finish_reason": o.finish_reason} for o in outs]

    def close(self):
        self.llm.close()


register_runner(RunnerDecl("llm.backbone", "autoregressive", LLMBackboneStage, inputs=("prompt", "audio", "image", "sampling"),
                           emits=("text", "token_ids", "finish_reason")))


class TalkerStage(Stage):
    """``tts.talker``: text (or templated token ids) → the codec frame matrix, through the Talker / CodePredictor loop of the
    speech pipeline in the artifact directory.  ``voice`` and ``sampling`` are optional inputs.  ``token_ids`` instead of
    ``text`` takes the bare ids a text decoder upstream generated (the thinker → talker hand-off of an audio-out
    deployment) and wraps them in the speech prompt's template."""

    def __init__(self, cfg: StageConfig, root: str, runtime=None):
        super().__init__(cfg, root)
        if runtime is None:
            from .tts import load_tts
            runtime = load_tts(os.path.normpath(os.path.join(root, cfg.artifact)), cfg.config.get("device", "cpu"))
        self.runtime = runtime

    def run(self, batch):
        from .tts import TTSSampling
        out = []
        for r in batch:                                            # the frame loop holds one request at a time
            if "text" in r:
                text = r["text"]
                ids = self.runtime.tokenize(text) if isinstance(text, str) else list(text)
            else:
                ids = self.runtime.template_ids(r["token_ids"])
            sp = TTSSampling.from_dict({**self.cfg.config, **(r.get("sampling") or {})})
            codes, reason, _, _ = self.runtime.generate_codes(ids, r.get("voice"), r.get("language"), sp)
            out.append({"codes": codes, "finish_reason": reason})
        return out


class Code2WavStage(Stage):
    """``tts.code2wav``: codec frame matrix → 16-bit PCM bytes (the graph's audio terminal)."""

    def __init__(self, cfg: StageConfig, root: str, runtime=None):
        super().__init__(cfg, root)
        if runtime is None:
            from .tts import load_tts
            runtime = load_tts(os.path.normpath(os.path.join(root, cfg.artifact)), cfg.config.get("device", "cpu"))
        self.vocoder, self.device = runtime.code2wav, runtime.device

    def run(self, batch):
        from ..models.tts import pcm16_bytes
        out = []
        for r in batch:
            codes = r["codes"]
            wav = self.vocoder(codes.t().contiguous()[None].to(self.device))[0] if codes.shape[0] else codes.new_zeros(0).float()
            out.append({"audio": pcm16_bytes(wav)})
        return out


register_runner(RunnerDecl("tts.talker", "autoregressive", TalkerStage, inputs=("text", "token_ids", "voice", "language", "sampling"),
                           emits=("codes", "finish_reason")))
register_runner(RunnerDecl("tts.code2wav", "iterative", Code2WavStage, inputs=("codes",), emits=("audio",)))


# ---- parsing and validation ------------------------------------------------------------------------------------------

def parse_graph(obj: Dict[str, Any], root: str = ".") -> GraphConfig:
    if not isinstance(obj, dict):
        raise GraphConfigError("the graph file must hold a JSON object")
    g = _view(_ms.StageGraph.parse_text(json.dumps(obj), root))
    validate_graph(g)
    return g


def load_graph(path: str) -> GraphConfig:
    f = os.path.join(path, CONFIG_NAME) if os.path.isdir(path) else path
    with open(f, "r", encoding="utf-8") as fh:
        return parse_graph(json.load(fh), os.path.dirname(os.path.abspath(f)))


def validate_graph(g: GraphConfig, check_runners: bool = True) -> List[str]:
    """Structure checks (and, with ``check_runners``, agreement with the runner table); returns the execution order."""
    return list(_native_graph(g).validate(check_runners))


def one_stage_graph(max_batch: int = 8, has_audio: bool = False, has_image: bool = False) -> Dict[str, Any]:
    """The graph a plain LLM / VLM / ASR build gets: one backbone stage whose text is the terminal."""
    inputs = [{"name": "prompt", "from": "request:messages", "on_missing": "fail"},
              {"name": "sampling", "from": "request:sampling", "on_missing": "skip"}]
    if has_audio:
        inputs.append({"name": "audio", "from": "request:audio", "on_missing": "skip"})
    if has_image:
        inputs.append({"name": "image", "from": "request:image", "on_missing": "skip"})
    return {"schema_version": SCHEMA_VERSION, "terminals": ["llm:text"],
            "stages": [{"id": "llm", "runner": "llm.backbone", "artifact": ".", "kind": "autoregressive", "max_batch": max_batch,
                        "inputs": inputs, "emits": [{"id": "text", "kind": "text", "transport": "chunk_stream", "terminal": True},
                                                    {"id": "token_ids", "kind": "tokens", "transport": "chunk_stream"}]}]}


def audio_out_graph(llm_artifact: str = ".", tts_artifact: str = "tts", max_batch: int = 8, talker_config: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """The graph of an audio-out deployment: the text decoder answers, its generated ids go to the talker, the talker's codec
    frames to the vocoder.  Terminals: the answer's text and the speech; a request that asks for the text only never loads
    or runs the speech stages."""
    return {"schema_version": SCHEMA_VERSION, "terminals": ["thinker:text", "code2wav:audio"], "stages": [
        {"id": "thinker", "runner": "llm.backbone", "artifact": llm_artifact, "kind": "autoregressive", "max_batch": max_batch,
         "inputs": [{"name": "prompt", "from": "request:messages"}, {"name": "sampling", "from": "request:sampling", "on_missing": "skip"}],
         "emits": [{"id": "text", "kind": "text", "terminal": True}, {"id": "token_ids", "kind": "tokens"}]},
        {"id": "talker", "runner": "tts.talker", "artifact": tts_artifact, "kind": "autoregressive", "config": dict(talker_config or {}),
         "inputs": [{"name": "token_ids", "from": "thinker:token_ids"}, {"name": "voice", "from": "request:voice", "on_missing": "skip"}],
         "emits": [{"id": "codes", "kind": "codec"}]},
        {"id": "code2wav", "runner": "tts.code2wav", "artifact": tts_artifact, "kind": "iterative",
         "inputs": [{"name": "codes", "from": "talker:codes"}], "emits": [{"id": "audio", "kind": "audio", "terminal": True}]}]}


def write_graph(engine_dir: str, graph: Dict[str, Any]) -> str:
    parse_graph(graph, engine_dir)
    p = os.path.join(engine_dir, CONFIG_NAME)
    with open(p, "w", encoding="utf-8") as f:
        json.dump(graph, f, indent=2)
    return p


# ---- routing and execution -------------------------------------------------------------------------------------------

@dataclass
class Route:
    """What one request runs: the stages (in order), the terminals it will receive and why anything was left out."""
    stages: List[str]
    terminals: List[str]
    skipped: Dict[str, str] = field(default_factory=dict)
    error: Optional[str] = None


def _route_view(r) -> Route:
    return Route(list(r.stages), list(r.terminals), dict(r.skipped), r.error)


def plan_route(g: GraphConfig, request: Dict[str, Any], want: Optional[Sequence[str]] = None) -> Route:
    fields = {k for k, v in request.items() if v is not None}
    return _route_view(_ms.plan_route(_native_graph(g), fields, None if want is None else list(want)))


def _cohort_key(r: Dict[str, Any]) -> str:
    # settings that hold for a whole batch: requests that differ in them do not share a cohort
    return json.dumps([r.get("sampling"), r.get("voice")], sort_keys=True, default=str)


class MultiStageRuntime:
    """The native run loop with Python stage classes plugged in.  ``stages`` hands in stages that are already loaded;
    every other stage is built from the runner table on first use."""

    def __init__(self, graph: GraphConfig, stages: Optional[Dict[str, Stage]] = None):
        self.graph = graph
        self._stages: Dict[str, Stage] = dict(stages or {})
        self._native = _ms.MultiStageRuntime()
        self._native.load(_native_graph(graph), check_runners=stages is None)
        self.order = list(self._native.order)
        for sid, stage in self._stages.items():
            self._native.set_stage(sid, self._callable(stage))
        for runner in {s.runner for s in graph.stages}:
            self._native.set_factory(runner, self._factory)

    @staticmethod
    def _callable(stage: Stage) -> Callable:
        return lambda spec, batch: stage.run(batch)

    def _factory(self, spec, root: str) -> Callable:
        stage = _RUNNERS[spec.runner].factory(self.graph.stage(spec.id), root)
        self._stages[spec.id] = stage
        return self._callable(stage)

    @classmethod
    def load(cls, path: str) -> "MultiStageRuntime":
        return cls(load_graph(path))

    def _submit_all(self, requests: Sequence[Dict[str, Any]], want) -> None:
        self._native.discard_pending()
        for r in requests:
            fields = {k: v for k, v in r.items() if v is not None}
            idx, why = self._native.submit(fields, list(want) if want is not None else [], _cohort_key(r), None, True)
            if idx < 0:
                self._native.discard_pending()
                raise GraphConfigError(why)

    def cohorts(self, requests: Sequence[Dict[str, Any]], want, batch_size: int) -> List[Tuple[List[int], Route]]:
        """Group requests that run the same stages with the same batch-wide settings, in file order."""
        self._submit_all(requests, want)
        try:
            return [(list(members), _route_view(route)) for members, route in self._native.cohorts(batch_size)]
        finally:
            self._native.discard_pending()

    def run(self, requests: Sequence[Dict[str, Any]], want: Optional[Sequence[str]] = None, batch_size: int = 1) -> List[Dict[str, Any]]:
        self._submit_all(requests, want)
        self._native.run(batch_size)
        return [{"ok": r.ok, "error": r.error, "outputs": r.outputs, "stages": json.loads(r.stages_json)} for r in self._native.take()]

    def close(self) -> None:
        self._native.close()
        for s in self._stages.values():
            s.close()
        self._stages = {}
