"""HTTP surface on CPU: OpenAI / Anthropic routes, SSE streaming, auth, admission (429 / 503), config validation."""
import json
import threading

import pytest
import torch
from fastapi.testclient import TestClient

from tensorrt_edge_llm_b200.chat_template import ChatTemplate
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.llm import LLM
from tensorrt_edge_llm_b200.server.app import create_app
from tensorrt_edge_llm_b200.server.config import ApiConfig, ServerConfigError, parse_server_config
from tensorrt_edge_llm_b200.server.engine_client import AdmissionController, QueueFull, QueueTimeout


class ByteTokenizer:
    """One token per UTF-8 byte (ids 3..258); enough to drive the text routes."""

    def encode(self, text, add_special_tokens=False):
        return [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids, skip_special_tokens=True):
        return bytes((i - 3) % 256 for i in ids).decode("utf-8", "replace")

    def id_to_bytes(self, i):
        return bytes([(i - 3) % 256])


@pytest.fixture(scope="module")
def llm():
    cfg = tiny_llama_config(num_hidden_layers=2, dtype="float32")
    m = LLM(cfg, device="cpu", max_batch_size=4, max_input_len=256, max_kv_cache_capacity=320, page_size=16, tokenizer=ByteTokenizer(),
            enable_in_flight_batching=True)
    yield m
    m.close()


@pytest.fixture(scope="module")
def client(llm):
    return TestClient(create_app(llm, ApiConfig(served_model_name="tiny", api_key="sekret"), ChatTemplate()))


AUTH = {"Authorization": "Bearer sekret"}


def test_health_models_and_auth(client):
    h = client.get("/health").json()
    assert h["status"] == "healthy" and h["model"] == "tiny" and h["engine"]["serving"] and h["active_requests"] == 0
    caps = h["capabilities"]
    assert caps["chat"] and caps["in_flight_batching"] and not caps["speech"] and caps["input_modalities"] == ["text"]
    assert caps["max_batch_size"] == 4 and caps["max_input_len"] == 256 and caps["max_model_len"] == 320 and caps["speculative_method"] is None
    assert set(h["scheduling"]) >= {"submitted", "completed", "decode_steps", "admitted_mid_flight", "stalls_no_capacity"}
    assert client.get("/health/ready").json() == {"status": "ready", "active_requests": 0, "queued_requests": 0}
    assert client.get("/v1/models").status_code == 401
    assert client.get("/v1/models", headers={"x-api-key": "sekret"}).json()["data"][0]["id"] == "tiny"


def test_chat_completion_and_determinism(client):
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0}
    a = client.post("/v1/chat/completions", json=body, headers=AUTH).json()
    b = client.post("/v1/chat/completions", json=body, headers=AUTH).json()
    assert a["object"] == "chat.completion" and a["usage"]["completion_tokens"] == 6
    assert a["choices"][0]["token_ids"] == b["choices"][0]["token_ids"]
    assert a["choices"][0]["finish_reason"] in ("length", "stop")
    assert a["usage"]["prompt_tokens"] == len("<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n")


def test_chat_stream_matches_blocking(client):
    body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "count"}]}], "max_tokens": 5, "temperature": 0}
    want = client.post("/v1/chat/completions", json=body, headers=AUTH).json()
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True}, headers=AUTH) as r:
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
        events = [l[6:] for l in r.iter_lines() if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert chunks[-1]["usage"]["completion_tokens"] == 5 and chunks[-1]["choices"][0]["finish_reason"] is not None
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks)
    assert text == want["choices"][0]["message"]["content"]


def test_completions_with_token_ids_and_errors(client):
    r = client.post("/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 3, "temperature": 0}, headers=AUTH).json()
    assert len(r["choices"][0]["token_ids"]) == 3 and r["usage"]["prompt_tokens"] == 4
    assert client.post("/v1/completions", json={"max_tokens": 3}, headers=AUTH).status_code == 400
    too_long = client.post("/v1/completions", json={"prompt": list(range(3, 400)), "max_tokens": 1}, headers=AUTH)
    assert too_long.status_code == 400 and too_long.json()["error"]["code"] == "context_length_exceeded"
    assert client.post("/v1/chat/completions", json={"messages": []}, headers=AUTH).status_code == 400


def test_anthropic_messages_and_count(client):
    body = {"model": "tiny", "max_tokens": 4, "temperature": 0, "system": "be brief", "messages": [{"role": "user", "content": "hi"}]}
    r = client.post("/v1/messages", json=body, headers=AUTH).json()
    assert r["type"] == "message" and r["usage"]["output_tokens"] == 4 and r["stop_reason"] in ("max_tokens", "end_turn")
    n = client.post("/v1/messages/count_tokens", json=body, headers=AUTH).json()["input_tokens"]
    assert n == r["usage"]["input_tokens"]
    assert client.post("/v1/messages", json={"messages": [{"role": "user", "content": "x"}]}, headers=AUTH).status_code == 400
    with client.stream("POST", "/v1/messages", json={**body, "stream": True}, headers=AUTH) as s:
        kinds = [l[7:] for l in s.iter_lines() if l.startswith("event: ")]
    assert kinds[0] == "message_start" and kinds[-1] == "message_stop" and "content_block_delta" in kinds


def test_responses_route(client):
    r = client.post("/v1/responses", json={"input": "ping", "instructions": "pong", "max_output_tokens": 3, "temperature": 0}, headers=AUTH).json()
    assert r["object"] == "response" and r["usage"]["output_tokens"] == 3 and r["output"][0]["content"][0]["type"] == "output_text"
    # typed content parts and streaming events
    typed = {"input": [{"role": "user", "content": [{"type": "input_text", "text": "pi"}, {"type": "input_text", "text": "ng"}]}],
             "instructions": "pong", "max_output_tokens": 3, "temperature": 0}
    same = client.post("/v1/responses", json=typed, headers=AUTH).json()
    assert same["output_text"] == r["output_text"] and same["usage"]["input_tokens"] == r["usage"]["input_tokens"]
    with client.stream("POST", "/v1/responses", json={**typed, "stream": True}, headers=AUTH) as sresp:
        lines = [ln for ln in sresp.iter_lines() if ln]
    kinds = [ln[7:] for ln in lines if ln.startswith("event: ")]
    assert kinds[0] == "response.created" and kinds[-1] == "response.completed" and "response.output_text.done" in kinds
    import json as _js
    done = _js.loads([ln for ln in lines if ln.startswith("data: ")][-1][6:])
    assert done["response"]["status"] == "completed" and done["response"]["usage"]["output_tokens"] == 3
    assert client.post("/v1/responses", json={"input": [{"role": "user", "content": [{"type": "input_file"}]}]}, headers=AUTH).status_code == 400


def test_admission_controller_limits():
    ac = AdmissionController(slots=1, max_queued=1, timeout_s=0.2)
    ac.acquire()
    errs = []

    def waiter():
        try:
            ac.acquire()
            ac.release()
        except Exception as e:
            errs.append(e)

    t = threading.Thread(target=waiter)
    t.start()
    import time
    time.sleep(0.05)
    with pytest.raises(QueueFull):          # one runs, one waits, the third is refused
        ac.acquire()
    t.join()
    assert len(errs) == 1 and isinstance(errs[0], QueueTimeout)
    ac.release()
    ac.acquire()
    ac.release()
    assert ac.depth == (0, 0)


def test_server_config_validation():
    cfg = parse_server_config(["/ckpt", "--enable-in-flight-batching", "--scheduling-policy", "priority", "--preemption", "pause",
                               "--max-batch-size", "8", "--speculative-config", '{"method": "eagle3", "draft_model": "/d", "verify_tokens": 60}'])
    assert cfg.model.scheduling_dict()["preemption"] == "pause" and cfg.model.speculative_config.verify_tokens == 60
    with pytest.raises(ServerConfigError):
        parse_server_config(["/ckpt", "--scheduling-policy", "priority"])                   # needs IFB
    with pytest.raises(ServerConfigError):
        parse_server_config(["/ckpt", "--enable-in-flight-batching", "--preemption", "pause"])   # needs priority policy
    with pytest.raises(ServerConfigError):
        parse_server_config(["/ckpt", "--speculative-config", '{"method": "medusa"}'])
    with pytest.raises(ServerConfigError):
        parse_server_config(["/ckpt", "--max-kv-cache-capacity", "100", "--max-input-len", "200"])


def test_jinja_chat_template(tmp_path):
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({
        "bos_token": "<s>", "eos_token": {"content": "</s>"},
        "chat_template": "{{ bos_token }}{% for m in messages %}[{{ m.role }}] {{ m.content }}{{ eos_token }}{% endfor %}{% if add_generation_prompt %}[assistant]{% endif %}"}))
    t = ChatTemplate.load(str(tmp_path))
    assert t.apply([{"role": "user", "content": "a"}, {"role": "assistant", "content": [{"type": "text", "text": "b"}]}]) == \
        "<s>[user] a</s>[assistant] b</s>[assistant]"


def test_online_benchmark_against_the_app(llm):
    import asyncio

    import httpx

    from tensorrt_edge_llm_b200.benchmarks.online import percentile, run_workload, synthetic_workload
    assert percentile([1, 2, 3, 4], 50) == 2.5 and percentile([], 99) is None and percentile([5], 95) == 5
    app = create_app(llm, ApiConfig(served_model_name="tiny"), ChatTemplate())
    reqs = synthetic_workload(5, rate=50.0, prompt_len=4, max_tokens=4)
    assert reqs[0]["at_s"] == 0.0 and all(b["at_s"] >= a["at_s"] for a, b in zip(reqs, reqs[1:]))

    async def go():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://test") as client:
            return await run_workload(reqs, "http://test", "tiny", client=client)

    rep = asyncio.run(go())
    assert rep["requests"] == 5 and rep["completed"] == 5 and rep["failed"] == 0
    assert rep["output_tokens"] == 20 and rep["output_tokens_per_s"] > 0
    assert rep["ttft_s"]["p50"] is not None and rep["latency_s"]["p99"] >= rep["latency_s"]["p50"]


def test_chat_tool_call_and_reasoning_parsing(llm):
    """A completion forced (by a choice constraint) to be a wrapped call comes back as ``tool_calls``."""
    c = TestClient(create_app(llm, ApiConfig(served_model_name="tiny", reasoning_parser="think"), ChatTemplate()))
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object"}}}]
    call = '<think>look it up</think><tool_call>{"name": "get_weather", "arguments": {"city": "Paris"}}</tool_call>'
    body = {"messages": [{"role": "user", "content": "weather?"}], "tools": tools, "guided_choice": [call], "max_tokens": 120, "temperature": 0}
    r = c.post("/v1/chat/completions", json=body).json()
    msg = r["choices"][0]["message"]
    assert msg["tool_calls"][0]["function"] == {"name": "get_weather", "arguments": '{"city": "Paris"}'}
    assert msg["reasoning_content"] == "look it up" and msg["content"] is None
    assert r["choices"][0]["finish_reason"] == "tool_calls"
    assert c.post("/v1/chat/completions", json={**body, "tools": [{"type": "function"}]}).status_code == 400
    # with tool_choice "none" the text stays text
    r = c.post("/v1/chat/completions", json={**body, "tool_choice": "none"}).json()
    assert "tool_calls" not in r["choices"][0]["message"] and "<tool_call>" in r["choices"][0]["message"]["content"]


def test_logprobs_and_logit_bias(client, llm):
    body = {"prompt": [5, 9, 33], "max_tokens": 4, "temperature": 0, "logprobs": 3}
    r = client.post("/v1/completions", json=body, headers=AUTH).json()["choices"][0]
    lp = r["logprobs"]
    assert len(lp["token_logprobs"]) == 4 and lp["token_ids"] == r["token_ids"]
    for tid, chosen, top in zip(lp["token_ids"], lp["token_logprobs"], lp["top_logprobs"]):
        assert len(top) == 3 and chosen <= 0.0
        assert abs(max(top.values()) - chosen) < 1e-5 and str(tid) in top          # greedy: the chosen token leads the list
    # a large bias forces the token; a ban removes the otherwise greedy token
    forced = client.post("/v1/completions", json={**body, "logit_bias": {"77": 100}}, headers=AUTH).json()["choices"][0]
    assert forced["token_ids"] == [77] * 4 and all(abs(v) < 1e-3 for v in forced["logprobs"]["token_logprobs"])
    banned = client.post("/v1/completions", json={**body, "logit_bias": {str(r["token_ids"][0]): -100}}, headers=AUTH).json()["choices"][0]
    assert banned["token_ids"][0] != r["token_ids"][0]
    chat = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3, "temperature": 0,
                                                     "logprobs": True, "top_logprobs": 2}, headers=AUTH).json()["choices"][0]
    assert len(chat["logprobs"]["content"]) == 3 and len(chat["logprobs"]["content"][0]["top_logprobs"]) == 2
    assert client.post("/v1/completions", json={**body, "logprobs": 99}, headers=AUTH).status_code == 400
    # the static-batch path reports the same numbers
    from tensorrt_edge_llm_b200.runtime.llm import SamplingParams as SP
    static = LLM(llm.cfg, device="cpu", max_batch_size=2, max_input_len=64, max_kv_cache_capacity=128, page_size=16)
    static.model.load_state_dict(llm.model.state_dict())
    out = static.generate([[5, 9, 33]], SP(max_tokens=4, temperature=0.0, logprobs=3))[0]
    assert out.token_ids == r["token_ids"]
    assert all(abs(a["logprob"] - b) < 1e-4 for a, b in zip(out.logprobs, lp["token_logprobs"]))


def test_local_media_paths_need_an_allowed_directory(tmp_path):
    """A request cannot make the server read files unless a media directory was configured, and then only beneath it."""
    from tensorrt_edge_llm_b200.server import app as app_mod
    inside = tmp_path / "media"
    inside.mkdir()
    (inside / "a.ppm").write_bytes(b"P6\n1 1\n255\n\x01\x02\x03")
    secret = tmp_path / "secret.txt"
    secret.write_bytes(b"top secret")
    app_mod._MEDIA_ROOT["path"] = ""
    with pytest.raises(ValueError, match="disabled"):
        app_mod._media_bytes(str(inside / "a.ppm"))
    app_mod._MEDIA_ROOT["path"] = str(inside)
    try:
        assert app_mod._media_bytes(str(inside / "a.ppm")).startswith(b"P6")
        assert app_mod._media_bytes("file://" + str(inside / "a.ppm")).startswith(b"P6")
        for sneaky in (str(secret), str(inside / ".." / "secret.txt"), "file://" + str(secret)):
            with pytest.raises(ValueError, match="outside"):
                app_mod._media_bytes(sneaky)
        with pytest.raises(ValueError, match="not fetched"):
            app_mod._media_bytes("https://example.com/x.png")
        assert app_mod._media_bytes("data:image/png;base64,aGk=") == b"hi"
    finally:
        app_mod._MEDIA_ROOT["path"] = ""


def test_reference_command_line_flags_are_accepted():
    from tensorrt_edge_llm_b200.server.config import parse_server_config
    cfg = parse_server_config(["/ckpt", "--enable-in-flight-batching", "--enable-context-reuse", "--context-cache-max-records", "77",
                               "--context-cache-max-snapshots", "5", "--allowed-local-media-path", "/data/media", "--max-image-tokens-per-image", "256",
                               "--encoder-cache-budget-bytes", "1048576", "--cache-dir", "/tmp/x", "--clear-engine-cache",
                               "--speculative-config", '{"method": "dflash", "draft_model": "/d"}', "--spec-verify-tokens", "24", "--draft-top-k", "4"])
    cc, mc = cfg.model.context_cache_config, cfg.model.multimodal_config
    assert (cc.enabled, cc.max_records, cc.max_snapshots) == (True, 77, 5)
    assert (mc.max_image_tokens_per_image, mc.encoder_cache_budget_bytes) == (256, 1048576)
    assert cfg.api.allowed_local_media_path == "/data/media"
    sc = cfg.model.speculative_config
    assert (sc.method, sc.verify_tokens, sc.draft_top_k) == ("dflash", 24, 4)
