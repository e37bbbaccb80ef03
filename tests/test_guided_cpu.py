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


JSONISH = r"""
root   ::= "{" ws pair ("," ws pair)* "}"
pair   ::= string ":" ws value
string ::= "\"" [a-z]+ "\""
value  ::= [0-9]{1,3} | string | "true" | "false" | list
list   ::= "[" (value ("," value)*)? "]"
ws     ::= " "?
"""


def test_ebnf_matcher():
    from tensorrt_edge_llm_b200.runtime.grammar import EbnfMatcher, GrammarError
    m = EbnfMatcher(JSONISH)
    for good in ('{"a":1}', '{ "ab": "cd", "e":[1,22,"x",[true]]}', '{"k":[]}'):
        assert m.complete(good), good
        assert all(m.viable(good[:i]) for i in range(len(good) + 1))
    for bad in ('{"a":1', '{"A":1}', '{"a":1234}', '{"a":1}}', '["a"]'):
        assert not m.complete(bad), bad
    assert m.viable('{"a":12') and not m.viable('{"a":1234') and not m.viable("x") and not m.viable('{"a":1}x')
    # forced continuation (jump-forward): after an opening quote of a key nothing is forced, after `"a"` the colon is
    assert m.forced_continuation('{"a"') == ":"
    assert EbnfMatcher('root ::= "hello " name "!"\nname ::= [A-Z] [a-z]*').forced_continuation("") == "hello "
    # left recursion and nullable rules
    lr = EbnfMatcher('root ::= expr\nexpr ::= expr "+" term | term\nterm ::= [0-9]+ | "(" expr ")"\n')
    assert lr.complete("1+(2+33)+4") and lr.viable("1+(2+") and not lr.viable("1++") and not lr.complete("1+(2")
    assert EbnfMatcher('root ::= "a"* "b"?').complete("") and EbnfMatcher('root ::= ("ab" | "c"){2,}').complete("abcab")
    assert not EbnfMatcher('root ::= ("ab" | "c"){2,}').complete("c")
    for broken in ('start ::= "a"', 'root ::= missing', 'root ::= "abc', 'root ::= ("a"'):
        with pytest.raises(GrammarError):
            EbnfMatcher(broken)
    # the chart cache follows committed text and survives a probe that is not an extension
    m.commit('{"a":')
    assert m.viable('{"a": 7') and m.viable('{"b"') and m.complete('{"a":7}')


def test_structural_tag_matcher():
    from tensorrt_edge_llm_b200.runtime.grammar import GrammarError, StructuralTagMatcher
    spec = {"structures": [{"begin": "<function=get_weather>", "schema": {"type": "object", "properties": {"city": {"type": "string"}},
                                                                          "required": ["city"]}, "end": "</function>"},
                           {"begin": "<function=now>", "end": "</function>"}],
            "triggers": ["<function="]}
    m = StructuralTagMatcher(spec)
    ok = 'Sure. <function=get_weather>{"city": "Paris"}</function> and <function=now></function> done'
    assert m.complete(ok) and all(m.viable(ok[:i]) for i in range(len(ok) + 1))
    assert m.complete("no calls at all") and m.viable("text <fun")
    assert not m.viable("<function=unknown>") and not m.viable('<function=get_weather>{"town"')
    assert m.viable('<function=get_weather>{"city": "Pa') and not m.complete('<function=get_weather>{"city": "Pa')
    with pytest.raises(GrammarError):
        StructuralTagMatcher({"structures": [{"begin": "<x>", "end": "</x>"}], "triggers": ["<function="]})


def test_generate_under_a_grammar():
    """End to end on a random model: the output is a sentence of the grammar whatever the logits say."""
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.grammar import EbnfMatcher
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    g = 'root ::= "id-" [0-9]{3} ("-" [a-c]{2})?'
    cfg = tiny_llama_config(num_hidden_layers=1, vocab_size=300)
    cfg.eos_token_id = 2
    llm = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=32, max_kv_cache_capacity=64, page_size=16, tokenizer=ByteTokenizer(),
              enable_in_flight_batching=True)
    outs = llm.generate([[5, 6, 7], [9, 9]], SamplingParams(max_tokens=20, temperature=0.9, top_k=40, seed=3,
                                                            guided=GuidedDecodingParams("ebnf", grammar=g)))
    m = EbnfMatcher(g)
    for o in outs:
        assert m.complete(o.text), o.text
    llm.close()


def test_jump_forward_appends_forced_tokens_without_forward_passes():
    from tensorrt_edge_llm_b200.runtime.grammar import EbnfMatcher
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    g = 'root ::= "{\\"name\\": \\"" [a-z]{3} "\\", \\"ok\\": " ("true" | "false") "}"'
    cfg = tiny_llama_config(num_hidden_layers=1, vocab_size=300)
    cfg.eos_token_id = 2
    llm = LLM(cfg, device="cpu", max_batch_size=1, max_input_len=32, max_kv_cache_capacity=96, page_size=16, tokenizer=ByteTokenizer())
    calls = []
    step = llm.runner.step
    llm.runner.step = lambda seats, toks, **kw: (calls.append([len(t) for t in toks]), step(seats, toks, **kw))[1]
    plain = llm.generate([[5, 6]], SamplingParams(max_tokens=60, temperature=0.0, guided=GuidedDecodingParams("ebnf", grammar=g)))[0]
    n_plain = len(calls)
    calls.clear()
    fast = llm.generate([[5, 6]], SamplingParams(max_tokens=60, temperature=0.0,
                                                 guided=GuidedDecodingParams("ebnf", grammar=g, jump_forward=True)))[0]
    m = EbnfMatcher(g)
    assert m.complete(plain.text) and m.complete(fast.text) and fast.text == plain.text
    # only the three letters and the boolean's first letter are choices: everything else is appended in bulk
    assert llm.jump_forward_tokens >= 20 and len(calls) < n_plain / 3 and max(max(c) for c in calls) > 5
    llm.close()


def test_jump_forward_under_in_flight_batching():
    """The request engine's session emits grammar-forced tokens with the sampled one and feeds them as one multi-token row."""
    from tensorrt_edge_llm_b200.runtime.grammar import EbnfMatcher
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    g = 'root ::= "{\\"name\\": \\"" [a-z]{3} "\\", \\"ok\\": " ("true" | "false") "}"'
    cfg = tiny_llama_config(num_hidden_layers=1, vocab_size=300)
    cfg.eos_token_id = 2
    llm = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=32, max_kv_cache_capacity=96, page_size=16, tokenizer=ByteTokenizer(),
              enable_in_flight_batching=True)
    calls = []
    step = llm.runner.step
    llm.runner.step = lambda seats, toks, **kw: (calls.append([len(t) for t in toks]), step(seats, toks, **kw))[1]
    sp = lambda jf, **kw: SamplingParams(max_tokens=60, temperature=0.0, guided=GuidedDecodingParams("ebnf", grammar=g, jump_forward=jf), **kw)
    plain = llm.generate([[5, 6]], sp(False))[0]
    n_plain = len(calls)
    calls.clear()
    fast = llm.generate([[5, 6]], sp(True))[0]
    m = EbnfMatcher(g)
    assert m.complete(plain.text) and fast.text == plain.text and fast.finish_reason == plain.finish_reason
    assert llm.session.jump_forward_tokens >= 20 and len(calls) < n_plain / 3 and max(max(c) for c in calls) > 5
    # two requests in one batch, one of them without jump-forward, and a budget that ends inside a forced run
    before = llm.session.jump_forward_tokens
    a, b = llm.generate([[5, 6], [7, 8, 9]], sp(True))
    assert a.text == plain.text and m.complete(b.text)
    short = llm.generate([[5, 6]], SamplingParams(max_tokens=7, temperature=0.0,
                                                  guided=GuidedDecodingParams("ebnf", grammar=g, jump_forward=True)))[0]
    assert short.token_ids == plain.token_ids[:7] and short.finish_reason == "length"
    # a log-probability report keeps one row per token: such a request decodes token by token
    mark = llm.session.jump_forward_tokens
    lp_out = llm.generate([[5, 6]], sp(True, logprobs=1))[0]
    assert lp_out.text == plain.text and len(lp_out.logprobs) == len(lp_out.token_ids) and llm.session.jump_forward_tokens == mark > before
    llm.close()
