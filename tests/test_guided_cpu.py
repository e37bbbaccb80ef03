"""Guided decoding: matchers, bitmasks and constrained generation with a tiny model and a byte tokenizer."""
import json

import pytest
import torch

from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.guided import (GuidedDecoder, GuidedDecodingParams, _JsonObjectMatcher, generate_guided, make_matcher,
                                                   schema_to_regex)
from tensorrt_edge_llm_b200.runtime.llm import LLM


class ByteTokenizer:
    def encode(self, text, add_special_tokens=False):
        return [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids, skip_special_tokens=True):
        return bytes((i - 3) % 256 for i in ids).decode("utf-8", "replace")

    def id_to_bytes(self, i):
        return bytes([i - 3]) if 3 <= i < 259 else b""


@pytest.fixture(scope="module")
def llm():
    cfg = tiny_llama_config(num_hidden_layers=2, dtype="float32", vocab_size=259)
    cfg.eos_token_id = 2
    return LLM(cfg, device="cpu", max_batch_size=2, max_input_len=64, max_kv_cache_capacity=256, page_size=16, tokenizer=ByteTokenizer())


def test_json_matcher_prefixes_and_completion():
    m = _JsonObjectMatcher(max_depth=3)
    good = '{"a": [1, 2.5e3, true, null], "b": {"c": "x\\n"}}'
    for i in range(len(good) + 1):
        assert m.viable(good[:i]), good[:i]
    assert m.complete(good) and not m.complete(good[:-1]) and m.complete(" {} ")
    for bad in ('[1]', '{"a" 1}', '{"a": tru3}', '{,}', '{"a": 1}}', '{"a": {"b": {"c": {"d": 1}}}}', '{"a": "\x01"}'):
        assert not m.viable(bad), bad


def test_schema_regex_and_choice_matcher():
    import regex
    rx = schema_to_regex({"type": "object", "properties": {"name": {"type": "string"}, "n": {"type": "integer"},
                                                           "ok": {"type": "boolean"}, "kind": {"enum": ["a", "b"]}}})
    assert regex.fullmatch(rx, '{"name": "x y", "n": -12, "ok": true, "kind": "b"}')
    assert not regex.fullmatch(rx, '{"name": "x", "n": 1.5, "ok": true, "kind": "b"}')
    c = make_matcher(GuidedDecodingParams("choice", choices=["yes", "no", "maybe"]))
    assert c.viable("ma") and not c.viable("x") and c.complete("no") and not c.complete("n")
    with pytest.raises(ValueError):
        GuidedDecodingParams("ebnf")


def test_bitmask_marks_exactly_the_viable_tokens():
    tok = ByteTokenizer()
    dec = GuidedDecoder(GuidedDecodingParams("choice", choices=["cat", "car"]), GuidedDecoder.vocabulary(tok, 259), [2])
    bits = dec.bitmask()
    allowed = [t for t in range(259) if (int(bits[t // 32]) >> (t % 32)) & 1]
    assert allowed == [ord("c") + 3]
    for ch in "ca":
        dec.advance(ord(ch) + 3)
    bits = dec.bitmask()
    assert sorted(t for t in range(259) if (int(bits[t // 32]) >> (t % 32)) & 1) == sorted([ord("t") + 3, ord("r") + 3])
    dec.advance(ord("t") + 3)
    bits = dec.bitmask()
    assert [t for t in range(259) if (int(bits[t // 32]) >> (t % 32)) & 1] == [2]          # only end-of-sequence remains
    with pytest.raises(ValueError):
        dec.advance(ord("x") + 3)


def test_constrained_generation(llm):
    tok = llm.tokenizer
    out = tok.decode(generate_guided(llm, tok.encode("pick:"), GuidedDecodingParams("choice", choices=["alpha", "beta", "gamma"]), 16))
    assert out in ("alpha", "beta", "gamma")
    out = tok.decode(generate_guided(llm, tok.encode("id:"), GuidedDecodingParams("regex", pattern=r"[A-F][0-9]{3}-[a-z]{2}"), 16))
    import regex
    assert regex.fullmatch(r"[A-F][0-9]{3}-[a-z]{2}", out)
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}}}
    text = tok.decode(generate_guided(llm, tok.encode("json:"), GuidedDecodingParams("json_schema", json_schema=schema), 96))
    obj = json.loads(text)
    assert set(obj) == {"ok", "n"} and isinstance(obj["ok"], bool) and isinstance(obj["n"], int)
    # free-form JSON object: whatever the random model prefers, every prefix stays valid JSON
    ids = generate_guided(llm, tok.encode("x"), GuidedDecodingParams("json_object", max_depth=2), 24)
    assert _JsonObjectMatcher(2).viable(tok.decode(ids))


def test_server_response_format_and_guided_choice(llm):
    from fastapi.testclient import TestClient

    from tensorrt_edge_llm_b200.chat_template import ChatTemplate
    from tensorrt_edge_llm_b200.server.app import create_app
    client = TestClient(create_app(llm, None, ChatTemplate()))
    msgs = [{"role": "user", "content": "go"}]
    r = client.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 12, "guided_choice": ["left", "right"]}).json()
    assert r["choices"][0]["message"]["content"] in ("left", "right") and r["choices"][0]["finish_reason"] == "stop"
    schema = {"type": "object", "properties": {"go": {"type": "boolean"}}}
    r = client.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 40,
                                                  "response_format": {"type": "json_schema", "json_schema": {"schema": schema}}}).json()
    assert isinstance(json.loads(r["choices"][0]["message"]["content"])["go"], bool)
    assert client.post("/v1/chat/completions", json={"messages": msgs, "response_format": {"type": "json_schema"}}).status_code == 400
