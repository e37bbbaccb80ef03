"""Multimodal runner on CPU: image and audio rows spliced into the prompt, multimodal RoPE, encoder cache, pruning."""
import numpy as np
import torch

from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.models.audio import AudioConfig, AudioEncoder
from tensorrt_edge_llm_b200.models.vit import VisionConfig, VisionEncoder
from tensorrt_edge_llm_b200.runtime.llm import LLM
from tensorrt_edge_llm_b200.runtime.multimodal import MultimodalInputs, MultimodalRunner


def _llm(mrope):
    cfg = tiny_llama_config(num_hidden_layers=2, vocab_size=300, hidden_size=128, intermediate_size=256, num_attention_heads=2,
                            num_key_value_heads=1, head_dim=64)
    if mrope:
        cfg.mrope_section = [8, 12, 12]
    return LLM(cfg, device="cpu", max_batch_size=1, max_input_len=256, max_kv_cache_capacity=320, page_size=16)


def _encoders():
    v = VisionEncoder(VisionConfig(hidden_size=128, num_hidden_layers=1, num_attention_heads=2, intermediate_size=256, patch_size=4,
                                   image_size=16, out_hidden_size=128, spatial_merge=2, dtype="float32")).random_init(1, std=0.1)
    a = AudioEncoder(AudioConfig(n_mels=16, hidden_size=128, num_hidden_layers=1, num_attention_heads=2, intermediate_size=256,
                                 max_source_positions=50, avg_pool=2, out_hidden_size=128, dtype="float32")).random_init(2)
    return v, a


def test_image_and_audio_rows_replace_placeholders():
    llm = _llm(mrope=True)
    v, a = _encoders()
    mm = MultimodalRunner(llm, v, a, image_token_id=298, audio_token_id=299, cache_bytes=1 << 20)
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, (20, 24, 3), dtype=np.uint8)              # resized to the encoder's 16 x 16 input
    t = np.arange(16000) / 16000.0
    req = MultimodalInputs().text([5, 6, 7]).image(img).text([8, 9]).audio(0.3 * np.sin(2 * np.pi * 330 * t), 16000).text([10])
    ids, emb, pos3, delta = mm.build(req)
    assert ids.count(298) == 4 and ids.count(299) == 25 and len(ids) == 3 + 4 + 2 + 25 + 1 and emb.shape == (len(ids), 128)
    text_rows = llm.runner.embed_tokens([5, 6, 7])
    assert torch.equal(emb[:3], text_rows) and not torch.equal(emb[3], llm.runner.embed_tokens([0])[0])
    # the 2 x 2 image block shares its temporal position and spans two rows / columns; text after it continues at +2
    assert pos3[:, 3:7].tolist() == [[3, 3, 3, 3], [3, 3, 4, 4], [3, 4, 3, 4]] and pos3[:, 7].tolist() == [5, 5, 5]
    assert delta == -2
    out1 = mm.generate(req, max_tokens=5)
    assert mm.cache.misses == 2 and len(out1) == 5
    out2 = mm.generate(req, max_tokens=5)                                 # both encoders are served from the cache
    assert out2 == out1 and mm.cache.hits >= 2
    other = MultimodalInputs().text([5, 6, 7]).image(255 - img).text([8, 9]).audio(0.3 * np.sin(2 * np.pi * 330 * t), 16000).text([10])
    assert not torch.equal(mm.build(other)[1][3:7], emb[3:7])
    llm.close()


def test_pruning_shortens_the_prompt_and_plain_rope_decoders_work():
    llm = _llm(mrope=False)
    v, _ = _encoders()
    v8 = VisionEncoder(VisionConfig(hidden_size=128, num_hidden_layers=1, num_attention_heads=2, intermediate_size=256, patch_size=4,
                                    image_size=32, out_hidden_size=128, spatial_merge=2, dtype="float32")).random_init(1, std=0.1)
    img = np.zeros((32, 32, 3), dtype=np.uint8)                           # a flat image: its 16 rows are near-duplicates
    img[:8, :8] = 255
    full = MultimodalRunner(llm, v8, image_token_id=298)
    pruned = MultimodalRunner(llm, v8, image_token_id=298, visual_keep_ratio=0.5)
    req = MultimodalInputs().text([3, 4]).image(img).text([5])
    ids_f, _, p3, _ = full.build(req)
    ids_p, emb_p, _, _ = pruned.build(req)
    assert ids_f.count(298) == 16 and ids_p.count(298) == 8 and p3 is None and emb_p.shape[0] == len(ids_p)
    assert len(pruned.generate(req, max_tokens=3)) == 3
    llm.close()


def test_chat_route_with_image_and_audio_parts():
    import base64
    import io
    import wave
    from fastapi.testclient import TestClient
    from tensorrt_edge_llm_b200.chat_template import ChatTemplate
    from tensorrt_edge_llm_b200.server.app import create_app

    class Bytes:
        def encode(self, text, add_special_tokens=False):
            return [b + 3 for b in text.encode("utf-8")]

        def decode(self, ids, skip_special_tokens=True):
            return bytes((i - 3) % 256 for i in ids).decode("utf-8", "replace")
    llm = _llm(mrope=True)
    llm.tokenizer = Bytes()
    v, a = _encoders()
    mm = MultimodalRunner(llm, v, a, image_token_id=298, audio_token_id=299)
    ppm = b"P6\n8 8\n255\n" + bytes(range(192))
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(1); w.setsampwidth(2); w.setframerate(16000)
        w.writeframes((np.sin(np.arange(8000) / 20.0) * 8000).astype(np.int16).tobytes())
    msg = [{"role": "user", "content": [{"type": "text", "text": "look: "},
                                        {"type": "image_url", "image_url": {"url": "data:image/x-portable-pixmap;base64," + base64.b64encode(ppm).decode()}},
                                        {"type": "input_audio", "input_audio": {"data": base64.b64encode(buf.getvalue()).decode(), "format": "wav"}},
                                        {"type": "text", "text": " what is it?"}]}]
    c = TestClient(create_app(llm, chat_template=ChatTemplate(), multimodal=mm))
    r = c.post("/v1/chat/completions", json={"messages": msg, "max_tokens": 4})
    assert r.status_code == 200, r.text
    out = r.json()
    assert out["usage"]["completion_tokens"] == 4 and len(out["choices"][0]["token_ids"]) == 4
    plain = TestClient(create_app(llm, chat_template=ChatTemplate()))
    assert plain.post("/v1/chat/completions", json={"messages": msg, "max_tokens": 4}).status_code == 400
    bad = [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "https://example.com/x.png"}}]}]
    assert c.post("/v1/chat/completions", json={"messages": bad}).status_code == 400
    # transcription route: multipart upload of the clip, json or plain-text answer
    r = c.post("/v1/audio/transcriptions", files={"file": ("clip.wav", buf.getvalue(), "audio/wav")},
               data={"language": "en", "max_tokens": "5"})
    assert r.status_code == 200 and isinstance(r.json()["text"], str) and r.json()["usage"]["seconds"] == 0.5
    r = c.post("/v1/audio/transcriptions", files={"file": ("clip.wav", buf.getvalue(), "audio/wav")},
               data={"response_format": "text", "max_tokens": "3"})
    assert r.status_code == 200 and r.headers["content-type"].startswith("text/plain")
    assert c.post("/v1/audio/transcriptions", files={"file": ("clip.wav", b"not a wav", "audio/wav")}).status_code == 400
    assert c.post("/v1/audio/transcriptions", files={"file": ("clip.wav", buf.getvalue(), "audio/wav")},
                  data={"response_format": "srt"}).status_code == 400
    assert plain.post("/v1/audio/transcriptions", files={"file": ("clip.wav", buf.getvalue(), "audio/wav")}).status_code == 400
    assert c.get("/v1/voices").json() == {"object": "list", "data": []}
    assert c.post("/v1/audio/speech", json={"input": "hi", "voice": "x"}).status_code == 400
    llm.close()


def test_multimodal_requests_under_in_flight_batching():
    """With the request engine on, multimodal prompts join its steps (chunked, next to text requests) and give the same tokens
    as the static path."""
    import threading
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams
    cfg = _llm(mrope=True).cfg
    static = LLM(cfg, device="cpu", max_batch_size=3, max_input_len=256, max_kv_cache_capacity=320, page_size=16)
    v, a = _encoders()
    rng = np.random.default_rng(3)
    img = rng.integers(0, 255, (32, 32, 3), dtype=np.uint8)
    clip = (np.sin(np.arange(8000) / 15.0) * 0.3).astype(np.float32)
    reqs = [MultimodalInputs().text([3, 4, 5]).image(img).text([6, 7]),
            MultimodalInputs().text([8]).audio(clip, 16000).text([9, 10, 11]).image(img).text([12])]
    mm_static = MultimodalRunner(static, v, a, image_token_id=298, audio_token_id=299)
    want = [mm_static.generate(r, max_tokens=6) for r in reqs]
    text_want = static.generate([[20, 21, 22, 23]], SamplingParams(max_tokens=6, ignore_eos=True))[0].token_ids
    ifb = LLM(cfg, device="cpu", max_batch_size=3, max_input_len=256, max_kv_cache_capacity=320, page_size=16, enable_in_flight_batching=True,
              enable_prefix_cache=True, scheduling={"max_chunk_tokens": 16, "max_num_tokens": 48})
    mm = MultimodalRunner(ifb, v, a, image_token_id=298, audio_token_id=299)
    got = [None, None]
    th = [threading.Thread(target=lambda i=i: got.__setitem__(i, mm.generate(reqs[i], max_tokens=6))) for i in range(2)]
    for t in th:
        t.start()
    text_got = ifb.generate([[20, 21, 22, 23]], SamplingParams(max_tokens=6, ignore_eos=True))[0].token_ids
    for t in th:
        t.join()
    assert got == want and text_got == text_want
    # the same placeholder ids with another image must not reuse the first prompt's pages
    other = MultimodalInputs().text([3, 4, 5]).image(rng.integers(0, 255, (32, 32, 3), dtype=np.uint8)).text([6, 7])
    assert mm.generate(other, max_tokens=6) == mm_static.generate(other, max_tokens=6)
    assert ifb.session.mm_store == {}
    ifb.close()


def test_server_multimodal_chat_on_the_request_engine():
    """With in-flight batching the image request takes the ordinary chat path: same tokens streamed and not streamed."""
    import base64
    import json as js
    from fastapi.testclient import TestClient
    from tensorrt_edge_llm_b200.chat_template import ChatTemplate
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.server.app import create_app

    class Bytes:
        def encode(self, text, add_special_tokens=False):
            return [b + 3 for b in text.encode("utf-8")]

        def decode(self, ids, skip_special_tokens=True):
            return bytes((i - 3) % 256 for i in ids).decode("utf-8", "replace")

        def id_to_bytes(self, i):
            return bytes([(i - 3) % 256])
    cfg = _llm(mrope=True).cfg
    llm = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=256, max_kv_cache_capacity=320, page_size=16, tokenizer=Bytes(),
              enable_in_flight_batching=True)
    v, a = _encoders()
    mm = MultimodalRunner(llm, v, a, image_token_id=298, audio_token_id=299)
    c = TestClient(create_app(llm, chat_template=ChatTemplate(), multimodal=mm))
    ppm = b"P6\n8 8\n255\n" + bytes(range(192))
    msg = [{"role": "user", "content": [{"type": "text", "text": "look: "},
                                        {"type": "image_url", "image_url": {"url": "data:image/x-portable-pixmap;base64," + base64.b64encode(ppm).decode()}}]}]
    r = c.post("/v1/chat/completions", json={"messages": msg, "max_tokens": 5, "ignore_eos": True, "temperature": 0})
    assert r.status_code == 200, r.text
    full = r.json()
    assert full["usage"]["completion_tokens"] == 5 and full["usage"]["prompt_tokens"] > 16      # image rows count as prompt tokens
    with c.stream("POST", "/v1/chat/completions", json={"messages": msg, "max_tokens": 5, "ignore_eos": True, "temperature": 0, "stream": True}) as s:
        chunks = [js.loads(line[6:]) for line in s.iter_lines() if line.startswith("data: ") and line != "data: [DONE]"]
    usage = [ch["usage"] for ch in chunks if ch.get("usage")]
    finish = [ch["choices"][0]["finish_reason"] for ch in chunks if ch.get("choices") and ch["choices"][0].get("finish_reason")]
    assert finish == ["length"] and (not usage or usage[-1]["completion_tokens"] == 5)
    # the same request twice gives the same answer (random bytes do not survive a text comparison across the two framings)
    again = c.post("/v1/chat/completions", json={"messages": msg, "max_tokens": 5, "ignore_eos": True, "temperature": 0}).json()
    assert again["choices"][0]["message"]["content"] == full["choices"][0]["message"]["content"]
    bad = [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "data:image/png;base64," + base64.b64encode(b"nope").decode()}}]}]
    assert c.post("/v1/chat/completions", json={"messages": bad}).status_code == 400
    # Anthropic messages with an image block: same prompt rows, same answer
    amsg = [{"role": "user", "content": [{"type": "text", "text": "look: "},
                                         {"type": "image", "source": {"type": "base64", "media_type": "image/x-portable-pixmap",
                                                                      "data": base64.b64encode(ppm).decode()}}]}]
    r = c.post("/v1/messages", json={"messages": amsg, "max_tokens": 5, "temperature": 0})
    assert r.status_code == 200, r.text
    assert r.json()["usage"]["input_tokens"] == full["usage"]["prompt_tokens"]
    assert c.post("/v1/messages/count_tokens", json={"messages": amsg}).json()["input_tokens"] == full["usage"]["prompt_tokens"]
    llm.close()


def test_multimodal_request_on_a_speculative_deployment():
    """Media prompts share the engine with speculative text requests and decode token by token themselves."""
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams
    cfg = _llm(mrope=False).cfg
    dcfg = tiny_llama_config(num_hidden_layers=1, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_attention_heads=cfg.num_attention_heads,
                             num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, dtype=cfg.dtype)
    dcfg.draft_type, dcfg.eagle3_target_hidden_size = "eagle3", cfg.hidden_size
    static = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=256, max_kv_cache_capacity=320, page_size=16)
    v, a = _encoders()
    img = np.random.default_rng(5).integers(0, 255, (32, 32, 3), dtype=np.uint8)
    req = MultimodalInputs().text([3, 4, 5]).image(img).text([6, 7])
    want = MultimodalRunner(static, v, a, image_token_id=298, audio_token_id=299).generate(req, max_tokens=5)
    text_want = static.generate([[20, 21, 22, 23]], SamplingParams(max_tokens=8, ignore_eos=True))[0].token_ids
    spec = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=256, max_kv_cache_capacity=320, page_size=16, draft_model=dcfg,
               enable_in_flight_batching=True)
    mm = MultimodalRunner(spec, v, a, image_token_id=298, audio_token_id=299)
    assert mm.generate(req, max_tokens=5) == want
    assert spec.generate([[20, 21, 22, 23]], SamplingParams(max_tokens=8, ignore_eos=True))[0].token_ids == text_want
    spec.close()


def test_prepared_prompts_on_the_static_path_and_in_the_infer_command(tmp_path):
    """``LLM.generate`` takes a prepared multimodal prompt without the request engine too; ``trtedge infer`` builds one from
    messages that name an image file."""
    from tensorrt_edge_llm_b200.chat_template import ChatTemplate
    from tensorrt_edge_llm_b200.commands.infer import parse_request_file, run_requests
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams

    class Bytes:
        def encode(self, text, add_special_tokens=False):
            return [b + 3 for b in text.encode("utf-8")]

        def decode(self, ids, skip_special_tokens=True):
            return bytes((i - 3) % 256 for i in ids).decode("utf-8", "replace")
    llm = _llm(mrope=True)
    llm.tokenizer = Bytes()
    v, a = _encoders()
    mm = MultimodalRunner(llm, v, a, image_token_id=298, audio_token_id=299)
    img = np.random.default_rng(6).integers(0, 255, (32, 32, 3), dtype=np.uint8)
    req = MultimodalInputs().text([3, 4, 5]).image(img).text([6, 7])
    want = mm.generate(req, max_tokens=5)
    out = llm.generate([mm.prepare(req), [20, 21, 22]], SamplingParams(max_tokens=5, ignore_eos=True))
    assert out[0].token_ids == want and len(out[1].token_ids) == 5 and out[0].prompt_token_ids.count(298) > 0
    ppm = tmp_path / "frame.ppm"
    ppm.write_bytes(b"P6\n32 32\n255\n" + img.tobytes())
    body = {"max_generate_length": 4, "temperature": 0.0,
            "requests": [{"messages": [{"role": "user", "content": [{"type": "text", "text": "see "}, {"type": "image", "image": str(ppm)}]}]},
                         {"messages": [{"role": "user", "content": "plain"}]}]}
    res = run_requests(llm, ChatTemplate(), parse_request_file(body), mm)
    assert len(res) == 2 and res[0]["output_tokens"] == 4 and res[0]["input_tokens"] > res[1]["input_tokens"]
    import pytest
    from tensorrt_edge_llm_b200.commands.infer import RequestFileError
    with pytest.raises(RequestFileError):
        run_requests(llm, ChatTemplate(), parse_request_file(body), None)
    llm.close()
