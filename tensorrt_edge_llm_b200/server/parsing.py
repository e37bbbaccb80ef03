"""Assistant-output parsing for the chat routes: reasoning spans and tool calls.

Behaviour follows ``tensorrt_edgellm/server/parsing/reasoning.py`` (``<think>…</think>`` split, streaming
deltas that never leak half a marker) and ``tensorrt_edgellm/server/parsing/tool_calling.py`` (request
validation, wrapper-marker families, whole-text and streaming extraction, OpenAI ``tool_calls`` shape).

The design is one small scanner, :class:`_MarkerStream`, that splits an incoming character stream into
"outside" text and "inside a marker pair" text while holding back any suffix that could still grow
into a marker.  Reasoning and tool-call parsing are both instances of it; the whole-text functions feed
the complete string through the same scanner, so streaming and non-streaming results cannot drift.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

# --------------------------------------------------------------------------------------------------------------
# marker scanner


def _held_suffix(buf: str, tokens: Sequence[str]) -> int:
    """Length of the longest suffix of ``buf`` that is a proper prefix of one of ``tokens``."""
    best = 0
    for t in tokens:
        for n in range(min(len(t) - 1, len(buf)), best, -1):
            if buf.endswith(t[:n]):
                best = n
                break
    return best


class _MarkerStream:
    """Splits fed text into ``("out", s)`` / ``("open", marker)`` / ``("in", s)`` / ``("close", marker)`` pieces."""

    def __init__(self, opens: Sequence[str], closes: Sequence[str], start_inside: bool = False):
        self.opens, self.closes = tuple(opens), tuple(closes)
        self.inside = start_inside
        self.buf = ""

    def feed(self, text: str) -> List[Tuple[str, str]]:
        self.buf += text
        out: List[Tuple[str, str]] = []
        while self.buf:
            tokens = self.closes if self.inside else self.opens
            hit, at = None, len(self.buf)
            for t in tokens:
                i = self.buf.find(t)
                if i != -1 and (i < at or (i == at and hit is not None and len(t) > len(hit))):
                    hit, at = t, i
            if hit is None:
                keep = _held_suffix(self.buf, tokens)
                emit = self.buf[:len(self.buf) - keep]
                if emit:
                    out.append(("in" if self.inside else "out", emit))
                self.buf = self.buf[len(self.buf) - keep:]
                break
            if at:
                out.append(("in" if self.inside else "out", self.buf[:at]))
            out.append(("close" if self.inside else "open", hit))
            self.buf = self.buf[at + len(hit):]
            self.inside = not self.inside
        return out

    def flush(self) -> List[Tuple[str, str]]:
        out = [("in" if self.inside else "out", self.buf)] if self.buf else []
        self.buf = ""
        return out


# --------------------------------------------------------------------------------------------------------------
# reasoning


@dataclass
class ReasoningDelta:
    reasoning: str = ""
    content: str = ""


class StreamingReasoningParser:
    def __init__(self, start: str, end: str, starts_in_reasoning: bool):
        self._s = _MarkerStream((start,), (end,), start_inside=starts_in_reasoning)
        self._lead = True

    def _convert(self, pieces) -> List[ReasoningDelta]:
        out = []
        for kind, s in pieces:
            if kind == "in":
                out.append(ReasoningDelta(reasoning=s))
            elif kind == "out":
                if self._lead:                     # newlines right after the closing marker belong to neither side
                    s = s.lstrip("\n")
                    if not s:
                        continue
                    self._lead = False
                out.append(ReasoningDelta(content=s))
            elif kind == "close":
                self._lead = True
        return out

    def feed(self, text: str) -> List[ReasoningDelta]:
        return self._convert(self._s.feed(text))

    def flush(self) -> List[ReasoningDelta]:
        return self._convert(self._s.flush())


class ReasoningParser:
    """``<think>…</think>`` style reasoning split.  ``starts_in_reasoning`` covers chat templates that already put
    the opening marker into the prompt, so the completion begins inside the span."""

    def __init__(self, start_token: str = "<think>", end_token: str = "</think>", starts_in_reasoning: bool = False):
        self.start_token, self.end_token, self.starts_in_reasoning = start_token, end_token, starts_in_reasoning

    def stream(self) -> StreamingReasoningParser:
        return StreamingReasoningParser(self.start_token, self.end_token, self.starts_in_reasoning)

    def extract(self, text: str) -> Tuple[Optional[str], Optional[str]]:
        """``(reasoning, content)``; either is ``None`` when empty."""
        p = self.stream()
        ds = p.feed(text) + p.flush()
        reasoning = "".join(d.reasoning for d in ds).strip()
        content = "".join(d.content for d in ds).strip()
        return (reasoning or None), (content or None)


_REASONING_PARSERS = {
    "think": lambda: ReasoningParser(),
    "qwen3": lambda: ReasoningParser(),
    "deepseek-r1": lambda: ReasoningParser(starts_in_reasoning=True),
    "nemotron": lambda: ReasoningParser(),
}


def reasoning_parser_names() -> List[str]:
    return sorted(_REASONING_PARSERS) + ["auto", "none"]


def resolve_reasoning_parser(name: Optional[str], chat_template_source: str = "") -> Optional[ReasoningParser]:
    """``auto`` turns the parser on when the chat template itself mentions the markers."""
    if not name or name == "none":
        return None
    if name == "auto":
        if "<think>" not in chat_template_source and "</think>" not in chat_template_source:
            return None
        return ReasoningParser()
    if name not in _REASONING_PARSERS:
        raise ValueError(f"unknown reasoning parser {name!r}; known: {reasoning_parser_names()}")
    return _REASONING_PARSERS[name]()


# --------------------------------------------------------------------------------------------------------------
# tool calling: request side


@dataclass
class ToolConfig:
    tools: List[Dict[str, Any]] = field(default_factory=list)
    tool_choice: Any = "auto"

    @property
    def parse_output(self) -> bool:
        return bool(self.tools) and self.tool_choice != "none"

    @property
    def names(self) -> set:
        return {t["function"]["name"] for t in self.tools}

    @property
    def forced_name(self) -> Optional[str]:
        if isinstance(self.tool_choice, dict):
            return (self.tool_choice.get("function") or {}).get("name") or self.tool_choice.get("name")
        return None


def validate_tool_request(body: Dict[str, Any]) -> ToolConfig:
    """Checks ``tools`` / ``tool_choice`` / tool-role messages of a chat request; raises ``ValueError`` with the reason."""
    tools = body.get("tools") or []
    if not isinstance(tools, list):
        raise ValueError("tools must be a list")
    names = set()
    for i, t in enumerate(tools):
        if not isinstance(t, dict) or t.get("type", "function") != "function" or not isinstance(t.get("function"), dict):
            raise ValueError(f"tools[{i}] must be {{'type': 'function', 'function': {{...}}}}")
        fn = t["function"]
        name = fn.get("name")
        if not isinstance(name, str) or not re.fullmatch(r"[A-Za-z0-9_.\-]{1,64}", name):
            raise ValueError(f"tools[{i}].function.name is missing or malformed")
        if name in names:
            raise ValueError(f"duplicate tool name {name!r}")
        if "parameters" in fn and not isinstance(fn["parameters"], dict):
            raise ValueError(f"tools[{i}].function.parameters must be a JSON schema object")
        names.add(name)
    choice = body.get("tool_choice", "auto" if tools else "none")
    if isinstance(choice, str):
        if choice not in ("auto", "none", "required"):
            raise ValueError("tool_choice must be 'auto', 'none', 'required' or a named function")
        if choice == "required" and not tools:
            raise ValueError("tool_choice 'required' needs tools")
    elif isinstance(choice, dict):
        want = (choice.get("function") or {}).get("name") or choice.get("name")
        if want not in names:
            raise ValueError(f"tool_choice names unknown tool {want!r}")
    else:
        raise ValueError("tool_choice must be a string or an object")
    pending: set = set()
    for m in body.get("messages") or []:
        if not isinstance(m, dict):
            continue
        if m.get("role") == "assistant":
            for c in m.get("tool_calls") or []:
                if not isinstance(c, dict) or not isinstance(c.get("function"), dict) or "name" not in c["function"]:
                    raise ValueError("assistant tool_calls entries need function.name")
                if c.get("id"):
                    pending.add(c["id"])
        elif m.get("role") == "tool":
            tid = m.get("tool_call_id")
            if tid is not None and pending and tid not in pending:
                raise ValueError(f"tool message answers unknown tool_call_id {tid!r}")
    return ToolConfig(list(tools), choice)


# --------------------------------------------------------------------------------------------------------------
# tool calling: output side


@dataclass
class ToolCall:
    name: str
    arguments: str                     # JSON text
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])

    def to_openai(self, index: Optional[int] = None) -> Dict[str, Any]:
        d = {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}
        if index is not None:
            d["index"] = index
        return d


@dataclass
class ParsedAssistantOutput:
    content: str = ""
    reasoning: str = ""
    tool_calls: List[ToolCall] = field(default_factory=list)


# wrapper formats: (open markers, close markers, close may be missing at end of output)
_FAMILIES: Tuple[Tuple[Tuple[str, ...], Tuple[str, ...], bool], ...] = (
    (("<tool_call>",), ("</tool_call>",), False),
    (("<tool_calls>",), ("</tool_calls>",), False),
    (("<toolcall>",), ("</toolcall>",), False),
    (("<toolcalls>",), ("</toolcalls>",), False),
    (("<function_call>",), ("</function_call>",), False),
    (("<function_calls>",), ("</function_calls>",), False),
    (("[TOOL_CALLS]", "[TOOL_CALL]"), ("[/TOOL_CALLS]", "[/TOOL_CALL]"), True),
    (("<|python_tag|>",), ("<|eom_id|>", "<|eot_id|>"), True),
)
_OPENS = tuple(o for f in _FAMILIES for o in f[0]) + ("<function=",)
_CLOSE_OF = {o: f[1] for f in _FAMILIES for o in f[0]}
_CLOSE_OF["<function="] = ("</function>",)
_CLOSE_OPTIONAL = {o for f in _FAMILIES if f[2] for o in f[0]}


def _json_values(text: str) -> List[Any]:
    """Every top-level JSON value found in ``text`` (objects or arrays), skipping text between them."""
    dec, out, i = json.JSONDecoder(), [], 0
    while i < len(text):
        j = min((k for k in (text.find("{", i), text.find("[", i)) if k != -1), default=-1)
        if j == -1:
            break
        try:
            v, end = dec.raw_decode(text, j)
            out.append(v)
            i = end
        except json.JSONDecodeError:
            i = j + 1
    return out


def _calls_from_value(v: Any, allowed: Optional[set]) -> List[ToolCall]:
    if isinstance(v, list):
        return [c for e in v for c in _calls_from_value(e, allowed)]
    if not isinstance(v, dict):
        return []
    if isinstance(v.get("function"), dict):
        v = v["function"]
    name = v.get("name") or v.get("tool_name")
    if not isinstance(name, str) or (allowed is not None and name not in allowed):
        return []
    args = v.get("arguments", v.get("parameters", v.get("args", {})))
    if isinstance(args, str):
        try:
            json.loads(args)
            text = args
        except json.JSONDecodeError:
            text = json.dumps({"input": args})
    else:
        text = json.dumps(args if args is not None else {}, ensure_ascii=False)
    return [ToolCall(name, text)]


_PARAM_RE = re.compile(r"<parameter=([^>\s]+)>(.*?)(?:</parameter>|(?=<parameter=)|\Z)", re.S)


def _xml_function_call(head_and_body: str, allowed: Optional[set]) -> List[ToolCall]:
    """Body of ``<function=NAME>…</function>`` with ``<parameter=K>V</parameter>`` children (or one JSON object)."""
    name, _, body = head_and_body.partition(">")
    name = name.strip()
    if not name or (allowed is not None and name not in allowed):
        return []
    params = _PARAM_RE.findall(body)
    if not params:
        vals = _json_values(body)
        args = vals[0] if vals and isinstance(vals[0], dict) else {}
        return [ToolCall(name, json.dumps(args, ensure_ascii=False))]
    args: Dict[str, Any] = {}
    for k, raw in params:
        raw = raw.strip("\n")
        try:
            args[k] = json.loads(raw)
        except json.JSONDecodeError:
            args[k] = raw
    return [ToolCall(name, json.dumps(args, ensure_ascii=False))]


def _block_calls(open_marker: str, body: str, allowed: Optional[set]) -> List[ToolCall]:
    if open_marker == "<function=":
        return _xml_function_call(body, allowed)
    if "<function=" in body:                       # <tool_call><function=NAME>…</function></tool_call>
        out = []
        for part in body.split("<function=")[1:]:
            out += _xml_function_call(part.split("</function>")[0], allowed)
        return out
    calls = [c for v in _json_values(body) for c in _calls_from_value(v, allowed)]
    if not calls:
        m = re.match(r"\s*([A-Za-z0-9_.\-]+)\s*\n?\s*(\{.*)", body, re.S)       # NAME\n{json}
        if m and (allowed is None or m.group(1) in allowed):
            vals = _json_values(m.group(2))
            if vals and isinstance(vals[0], dict):
                calls = [ToolCall(m.group(1), json.dumps(vals[0], ensure_ascii=False))]
    return calls


class StreamingToolParser:
    """Incremental tool-call extraction: yields ``("content", text)`` and ``("tool_call", ToolCall)`` events.

    Text outside wrapper markers streams through immediately (minus a held-back suffix that may become a
    marker); a wrapped block is released as calls once its closing marker (or the end of output) arrives.
    A block that yields no valid call is returned as content, so nothing the model said is lost."""

    def __init__(self, tool_config: ToolConfig):
        self.cfg = tool_config
        self.allowed = tool_config.names or None
        self._buf = ""
        self._open: Optional[str] = None
        self._body = ""
        self._any_content = False
        self.calls: List[ToolCall] = []

    def _emit_block(self, closed_with: str) -> List[Tuple[str, Any]]:
        calls = _block_calls(self._open, self._body, self.allowed)
        ev: List[Tuple[str, Any]] = []
        if calls:
            for c in calls:
                self.calls.append(c)
                ev.append(("tool_call", c))
        else:
            ev.append(("content", self._open + self._body + closed_with))
        self._open, self._body = None, ""
        return ev

    def feed(self, text: str) -> List[Tuple[str, Any]]:
        self._buf += text
        ev: List[Tuple[str, Any]] = []
        while self._buf:
            if self._open is None:
                hit, at = None, len(self._buf)
                for t in _OPENS:
                    i = self._buf.find(t)
                    if i != -1 and (i < at or (i == at and len(t) > len(hit or ""))):
                        hit, at = t, i
                if hit is None:
                    keep = _held_suffix(self._buf, _OPENS)
                    emit = self._buf[:len(self._buf) - keep]
                    if emit:
                        ev.append(("content", emit))
                    self._buf = self._buf[len(self._buf) - keep:]
                    break
                if at:
                    ev.append(("content", self._buf[:at]))
                self._open, self._buf = hit, self._buf[at + len(hit):]
            else:
                closes = _CLOSE_OF[self._open]
                hit, at = None, len(self._buf)
                for t in closes:
                    i = self._buf.find(t)
                    if i != -1 and i < at:
                        hit, at = t, i
                if hit is None:
                    keep = _held_suffix(self._buf, closes)
                    self._body += self._buf[:len(self._buf) - keep]
                    self._buf = self._buf[len(self._buf) - keep:]
                    break
                self._body += self._buf[:at]
                self._buf = self._buf[at + len(hit):]
                ev += self._emit_block(hit)
        return self._filter(ev)

    def flush(self) -> List[Tuple[str, Any]]:
        ev: List[Tuple[str, Any]] = []
        if self._open is not None:
            self._body += self._buf
            self._buf = ""
            ev += self._emit_block("")
        elif self._buf:
            ev.append(("content", self._buf))
            self._buf = ""
        return self._filter(ev)

    def _filter(self, ev):
        out = []
        for kind, v in ev:
            if kind == "content":
                if not self._any_content and not v.strip():
                    continue                        # leading blank lines around tool blocks carry nothing
                self._any_content = True
            out.append((kind, v))
        return out


def _bare_json_calls(text: str, allowed: Optional[set]) -> Tuple[List[ToolCall], str]:
    """A completion that is nothing but JSON call objects (Llama-3 style, no wrapper)."""
    s = text.strip()
    if not s or s[0] not in "{[":
        return [], text
    dec = json.JSONDecoder()
    calls, i = [], 0
    while i < len(s):
        while i < len(s) and s[i] in " \t\r\n;,":
            i += 1
        if i >= len(s):
            break
        try:
            v, i = dec.raw_decode(s, i)
        except json.JSONDecodeError:
            return [], text
        got = _calls_from_value(v, allowed)
        if not got:
            return [], text
        calls += got
    return calls, ""


def parse_assistant_output(text: str, tool_config: Optional[ToolConfig] = None,
                           reasoning_parser: Optional[ReasoningParser] = None) -> ParsedAssistantOutput:
    """Whole-text parse: reasoning span first, then tool calls out of the remaining content."""
    out = ParsedAssistantOutput()
    if reasoning_parser is not None:
        r, c = reasoning_parser.extract(text)
        out.reasoning, text = r or "", c or ""
    if tool_config is None or not tool_config.parse_output:
        out.content = text
        return out
    p = StreamingToolParser(tool_config)
    ev = p.feed(text) + p.flush()
    content = "".join(v for k, v in ev if k == "content")
    out.tool_calls = [v for k, v in ev if k == "tool_call"]
    if not out.tool_calls:
        out.tool_calls, content = _bare_json_calls(content, tool_config.names or None)
    forced = tool_config.forced_name
    if forced:
        out.tool_calls = [c for c in out.tool_calls if c.name == forced]
    out.content = content.strip() if out.tool_calls else content
    return out


class StreamingAssistantOutputParser:
    """Reasoning split chained into the tool parser; emits dict events ``{"type": "reasoning"|"content"|"tool_call", …}``."""

    def __init__(self, tool_config: Optional[ToolConfig] = None, reasoning_parser: Optional[ReasoningParser] = None):
        self._r = reasoning_parser.stream() if reasoning_parser is not None else None
        self._t = StreamingToolParser(tool_config) if tool_config is not None and tool_config.parse_output else None
        self._n_calls = 0

    def _tools(self, text: str, last: bool = False) -> List[Dict[str, Any]]:
        if self._t is None:
            return [{"type": "content", "text": text}] if text else []
        ev = self._t.feed(text) if text else []
        if last:
            ev += self._t.flush()
        out = []
        for kind, v in ev:
            if kind == "content":
                out.append({"type": "content", "text": v})
            else:
                out.append({"type": "tool_call", "index": self._n_calls, "call": v})
                self._n_calls += 1
        return out

    def _route(self, deltas: Iterable[ReasoningDelta]) -> List[Dict[str, Any]]:
        out = []
        for d in deltas:
            if d.reasoning:
                out.append({"type": "reasoning", "text": d.reasoning})
            if d.content:
                out += self._tools(d.content)
        return out

    def feed(self, text: str) -> List[Dict[str, Any]]:
        if self._r is None:
            return self._tools(text)
        return self._route(self._r.feed(text))

    def flush(self) -> List[Dict[str, Any]]:
        out = self._route(self._r.flush()) if self._r is not None else []
        return out + self._tools("", last=True)

    @property
    def saw_tool_call(self) -> bool:
        return self._n_calls > 0
