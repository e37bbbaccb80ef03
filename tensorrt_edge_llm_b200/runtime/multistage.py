"""Multi-stage runtime: a JSON-described graph of stages (LLM backbone, encoders, talker, vocoder …) run per cohort.

Follows ``cpp/runtime/multiStage/`` (``multiStageRuntime``, ``route``, ``stageConfig``, stage registry and factories)
and ``docs/source/developer_guide/software-design/multi-stage-graph.md``: ``multistage_config.json`` lists stages
(``id``, ``runner``, ``artifact``, ``kind``, ``inputs[{name, from, on_missing}]``, ``emits[{id, kind, transport,
terminal}]``) and ``terminals``; a request runs only the stages whose inputs it can supply and whose outputs reach a
requested terminal; requests that run the same stages form a cohort of at most ``max_batch``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Set, Tuple

SCHEMA_VERSION = 1
CONFIG_NAME = "multistage_config.json"
_ON_MISSING = ("fail", "skip", "prune")


class GraphConfigError(ValueError):
    pass


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

    def stage(self, sid: str) -> StageConfig:
        for s in self.stages:
            if s.id == sid:
                return s
        raise KeyError(sid)


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


# ---- parsing and validation ------------------------------------------------------------------------------------------

def parse_graph(obj: Dict[str, Any], root: str = ".") -> GraphConfig:
    if not isinstance(obj, dict):
        raise GraphConfigError("the graph file must hold a JSON object")
    if obj.get("schema_version") != SCHEMA_VERSION:
        raise GraphConfigError(f"schema_version must be {SCHEMA_VERSION}")
    stages: List[StageConfig] = []
    for i, s in enumerate(obj.get("stages") or []):
        try:
            ins = [InputPort(p["name"], p["from"], p.get("on_missing", "fail")) for p in s.get("inputs", [])]
            ems = [EmitPort(e["id"], e.get("kind", "tensor"), e.get("transport", "chunk_stream"), bool(e.get("terminal", False)))
                   for e in s.get("emits", [])]
            stages.append(StageConfig(s["id"], s["runner"], s.get("artifact", "."), s.get("kind", "autoregressive"), ins, ems,
                                      int(s.get("max_batch", 0)), int(s.get("max_seq", 0)), dict(s.get("config", {}))))
        except (KeyError, TypeError) as e:
            raise GraphConfigError(f"stages[{i}] is missing {e}") from None
    g = GraphConfig(stages, list(obj.get("terminals") or []), root)
    validate_graph(g)
    return g


def load_graph(path: str) -> GraphConfig:
    f = os.path.join(path, CONFIG_NAME) if os.path.isdir(path) else path
    with open(f, "r", encoding="utf-8") as fh:
        return parse_graph(json.load(fh), os.path.dirname(os.path.abspath(f)))


def _topological(g: GraphConfig) -> List[str]:
    deps = {s.id: {p.ref[0] for p in s.inputs if not p.from_request} for s in g.stages}
    order: List[str] = []
    while deps:
        ready = sorted(k for k, d in deps.items() if not (d - set(order)))
        if not ready:
            raise GraphConfigError(f"the stages {sorted(deps)} form a cycle")
        for k in ready:
            order.append(k)
            del deps[k]
    return order


def validate_graph(g: GraphConfig, check_runners: bool = True) -> List[str]:
    """Structure checks (and, with ``check_runners``, agreement with the runner table); returns the execution order."""
    if not g.stages:
        raise GraphConfigError("a graph needs at least one stage")
    ids = [s.id for s in g.stages]
    if len(set(ids)) != len(ids):
        raise GraphConfigError("stage ids must be unique")
    ports = {(s.id, e.id) for s in g.stages for e in s.emits}
    for s in g.stages:
        if len({e.id for e in s.emits}) != len(s.emits):
            raise GraphConfigError(f"stage {s.id}: duplicate output port")
        for p in s.inputs:
            if p.on_missing not in _ON_MISSING:
                raise GraphConfigError(f"stage {s.id}: on_missing must be one of {_ON_MISSING}")
            if ":" not in p.source:
                raise GraphConfigError(f"stage {s.id}: input {p.name!r} needs a source of the form <stage>:<port> or request:<field>")
            if not p.from_request and p.ref not in ports:
                raise GraphConfigError(f"stage {s.id}: input {p.name!r} reads {p.source!r}, which no stage emits")
        if check_runners:
            decl = _RUNNERS.get(s.runner)
            if decl is None:
                raise GraphConfigError(f"stage {s.id}: unknown runner {s.runner!r}; known: {runner_names()}")
            if decl.kind != s.kind:
                raise GraphConfigError(f"stage {s.id}: runner {s.runner} is {decl.kind}, the graph says {s.kind}")
            bad_in = [p.name for p in s.inputs if decl.inputs and p.name not in decl.inputs]
            bad_out = [e.id for e in s.emits if decl.emits and e.id not in decl.emits]
            if bad_in or bad_out:
                raise GraphConfigError(f"stage {s.id}: runner {s.runner} has no input {bad_in} / output {bad_out}")
    marked = sorted(f"{s.id}:{e.id}" for s in g.stages for e in s.emits if e.terminal)
    for t in g.terminals:
        a, _, b = t.partition(":")
        if (a, b) not in ports:
            raise GraphConfigError(f"terminal {t!r} is not an output of any stage")
    if sorted(g.terminals) != marked:
        raise GraphConfigError(f"terminals {sorted(g.terminals)} differ from the outputs marked terminal {marked}")
    return _topological(g)


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


def plan_route(g: GraphConfig, request: Dict[str, Any], want: Optional[Sequence[str]] = None) -> Route:
    order = _topological(g)
    want = list(want) if want is not None else list(g.terminals)
    runnable: Set[str] = set()
    skipped: Dict[str, str] = {}
    for sid in order:
        s = g.stage(sid)
        why = None
        for p in s.inputs:
            present = (p.ref[1] in request and request[p.ref[1]] is not None) if p.from_request else p.ref[0] in runnable
            if not present and p.on_missing != "skip":
                why = f"input {p.name!r} ({p.source}) is missing"
                break
        if why is None:
            runnable.add(sid)
        else:
            skipped[sid] = why
    # keep only what reaches a requested terminal
    needed: Set[str] = set()
    frontier = [t.partition(":")[0] for t in want]
    while frontier:
        sid = frontier.pop()
        if sid in needed or sid not in runnable:
            continue
        needed.add(sid)
        frontier += [p.ref[0] for p in g.stage(sid).inputs if not p.from_request and p.ref[0] in runnable]
    got = [t for t in want if t.partition(":")[0] in needed]
    missing = [t for t in want if t not in got]
    err = None
    if missing:
        err = "; ".join(f"{t} needs stage {t.partition(':')[0]}: {skipped.get(t.partition(':')[0], 'an upstream stage cannot run')}" for t in missing)
    return Route([sid for sid in order if sid in needed], got, skipped, err)


class MultiStageRuntime:
    def __init__(self, graph: GraphConfig, stages: Optional[Dict[str, Stage]] = None):
        self.graph = graph
        self.order = validate_graph(graph, check_runners=stages is None)
        self._stages: Dict[str, Stage] = dict(stages or {})

    @classmethod
    def load(cls, path: str) -> "MultiStageRuntime":
        return cls(load_graph(path))

    def _stage(self, sid: str) -> Stage:
        if sid not in self._stages:                      # stages load on first use: a text-only run never loads the vocoder
            cfg = self.graph.stage(sid)
            self._stages[sid] = _RUNNERS[cfg.runner].factory(cfg, self.graph.root)
        return self._stages[sid]

    def cohorts(self, requests: Sequence[Dict[str, Any]], want, batch_size: int) -> List[Tuple[List[int], Route]]:
        """Group requests that run the same stages with the same batch-wide settings, in file order."""
        cap = batch_size
        for s in self.graph.stages:
            if s.max_batch:
                cap = min(cap, s.max_batch)
        groups: List[Tuple[tuple, List[int], Route]] = []
        for i, r in enumerate(requests):
            route = plan_route(self.graph, r, want)
            key = (tuple(route.stages), tuple(route.terminals), json.dumps(r.get("sampling"), sort_keys=True), r.get("voice"))
            for k, idx, _ in groups:
                if k == key and len(idx) < max(cap, 1):
                    idx.append(i)
                    break
            else:
                groups.append((key, [i], route))
        return [(idx, route) for _, idx, route in groups]

    def run(self, requests: Sequence[Dict[str, Any]], want: Optional[Sequence[str]] = None, batch_size: int = 1) -> List[Dict[str, Any]]:
        results: List[Dict[str, Any]] = [{} for _ in requests]
        for idx, route in self.cohorts(requests, want, batch_size):
            values: List[Dict[Tuple[str, str], Any]] = [{} for _ in idx]
            detail: Dict[str, Any] = {sid: {"ran": False, "reason": why} for sid, why in route.skipped.items()}
            error = route.error
            for sid in route.stages:
                cfg = self.graph.stage(sid)
                batch = []
                for j, i in enumerate(idx):
                    ins = {}
                    for p in cfg.inputs:
                        src = requests[i].get(p.ref[1]) if p.from_request else values[j].get(p.ref)
                        if src is not None:
                            ins[p.name] = src
                    batch.append(ins)
                try:
                    outs = self._stage(sid).run(batch)
                    for j, o in enumerate(outs):
                        for port, v in o.items():
                            values[j][(sid, port)] = v
                    detail[sid] = {"ran": True, "batch": len(idx)}
                except Exception as e:       # a failing stage fails its cohort, not the run
                    error = f"stage {sid}: {type(e).__name__}: {e}"
                    detail[sid] = {"ran": False, "reason": error}
                    break
            for j, i in enumerate(idx):
                out = {t: values[j].get(tuple(t.split(":", 1))) for t in route.terminals}
                ok = error is None and all(v is not None for v in out.values())
                results[i] = {"ok": ok, "error": None if ok else (error or "a terminal produced nothing"), "outputs": out, "stages": detail}
        return results

    def close(self) -> None:
        for s in self._stages.values():
            s.close()
        self._stages = {}
