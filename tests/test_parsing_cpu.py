"""Reasoning / tool-call parsing: whole text, streaming at every split point, request validation, the chat route."""
import json

import pytest

from tensorrt_edge_llm_b200.server import parsing as P

TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}},
         {"type": "function", "function": {"name": "add", "parameters": {"type": "object"}}}]
CFG = P.ToolConfig(TOOLS, "auto")


def test_reasoning_extract_and_stream_split_points():
    rp = P.ReasoningParser()
    text = "<think>\nstep one\nstep two\n</think>\n\nThe answer is 4."
    assert rp.extract(text) == ("step one\nstep two", "The answer is 4.")
    assert rp.extract("plain") == (None, "plain")
    assert P.ReasoningParser(starts_in_reasoning=True).extract("hidden</think>shown") == ("hidden", "shown")
    for cut in range(1, len(text)):
        s = rp.stream()
        ds = s.feed(text[:cut]) + s.feed(text[cut:]) + s.flush()
        assert "".join(d.reasoning for d in ds).strip() == "step one\nstep two"
        assert "".join(d.content for d in ds) == "The answer is 4."
        assert all("<" not in d.reasoning and "<" not in d.content for d in ds)      # no marker fragment leaks
    assert P.resolve_reasoning_parser("auto", "{{ '<think>' }}") is not None
    assert P.resolve_reasoning_parser("auto", "no markers") is None and P.resolve_reasoning_parser("none") is None
    with pytest.raises(ValueError):
        P.resolve_reasoning_parser("nope")


@pytest.mark.parametrize("text,calls,content", [
    ('Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>', [("get_weather", {"city": "Paris"})], "Let me check."),
    ('<tool_call>{"name": "add", "arguments": {"a": 1, "b": 2}}</tool_call><tool_call>{"name": "add", "arguments": {"a": 3, "b": 4}}</tool_call>',
     [("add", {"a": 1, "b": 2}), ("add", {"a": 3, "b": 4})], ""),
    ('[TOOL_CALLS][{"name": "get_weather", "arguments": {"city": "Rome"}}]', [("get_weather", {"city": "Rome"})], ""),
    ('<function=get_weather>\n<parameter=city>\nOslo\n</parameter>\n</function>', [("get_weather", {"city": "Oslo"})], ""),
    ('<tool_call>\n<function=add>\n<parameter=a>1</parameter>\n<parameter=b>[2, 3]</parameter>\n</function>\n</tool_call>', [("add", {"a": 1, "b": [2, 3]})], ""),
    ('{"name": "get_weather", "parameters": {"city": "Lima"}}', [("get_weather", {"city": "Lima"})], ""),
    ('<function_call>{"name": "add", "arguments": "{\\"a\\": 5}"}</function_call>', [("add", {"a": 5})], ""),
    ('no tools here, just {"braces": 1}', [], 'no tools here, just {"braces": 1}'),
    ('<tool_call>{"name": "unknown_tool", "arguments": {}}</tool_call>', [], '<tool_call>{"name": "unknown_tool", "arguments": {}}</tool_call>'),
])
def test_tool_call_formats_whole_and_streaming(text, calls, content):
    out = P.parse_assistant_output(text, CFG)
    assert [(c.name, json.loads(c.arguments)) for c in out.tool_calls] == calls
    assert out.content == content
    if text.lstrip().startswith("{"):
        return                                           # bare JSON is recognised on the finished text only
    for cut in range(1, len(text)):
        sp = P.StreamingAssistantOutputParser(CFG)
        ev = sp.feed(text[:cut]) + sp.feed(text[cut:]) + sp.flush()
        got = [(e["call"].name, json.loads(e["call"].arguments)) for e in ev if e["type"] == "tool_call"]
        assert got == calls
        assert [e["index"] for e in ev if e["type"] == "tool_call"] == list(range(len(calls)))
        assert "".join(e["text"] for e in ev if e["type"] == "content").strip() == content


def test_reasoning_then_tool_call_and_choice_rules():
    text = '<think>need weather</think>\n<tool_call>{"name": "get_weather", "arguments": {"city": "Kyiv"}}</tool_call>'
    out = P.parse_assistant_output(text, CFG, P.ReasoningParser())
    assert out.reasoning == "need weather" and out.content == "" and out.tool_calls[0].name == "get_weather"
    assert out.tool_calls[0].to_openai(0)["function"]["arguments"] == '{"city": "Kyiv"}'
    none = P.parse_assistant_output(text, P.ToolConfig(TOOLS, "none"))
    assert not none.tool_calls and "<tool_call>" in none.content
    forced = P.ToolConfig(TOOLS, {"type": "function", "function": {"name": "add"}})
    assert P.parse_assistant_output(text, forced).tool_calls == []


def test_validate_tool_request():
    ok = P.validate_tool_request({"tools": TOOLS, "messages": [
        {"role": "assistant", "tool_calls": [{"id": "call_1", "function": {"name": "add", "arguments": "{}"}}]},
        {"role": "tool", "tool_call_id": "call_1", "content": "3"}]})
    assert ok.parse_output and ok.names == {"get_weather", "add"}
    assert not P.validate_tool_request({}).parse_output
    for bad in ({"tools": "x"}, {"tools": [{"type": "function"}]}, {"tools": TOOLS + TOOLS[:1]}, {"tools": TOOLS, "tool_choice": "sometimes"},
                {"tool_choice": "required"}, {"tools": TOOLS, "tool_choice": {"type": "function", "function": {"name": "nope"}}},
                {"tools": [{"type": "function", "function": {"name": "bad name!"}}]},
                {"tools": TOOLS, "messages": [{"role": "assistant", "tool_calls": [{"id": "a", "function": {"name": "add"}}]},
                                              {"role": "tool", "tool_call_id": "b", "content": ""}]}):
        with pytest.raises(ValueError):
            P.validate_tool_request(bad)
