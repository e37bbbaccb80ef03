"""Speech generation: prompt layout, the Talker / CodePredictor frame loop against a cache-free restatement, the
vocoder's shapes and chunked decoding, the artefact directory and the audio container."""
import io
import wave

import pytest
import torch

from tensorrt_edge_llm_b200.models.tts import Code2Wav, Code2WavConfig, TTSConfig, pcm16_bytes, wav_file_bytes
from tensorrt_edge_llm_b200.runtime import tts as T

TEXT = [1, 2, 3, 10, 11, 12, 13, 14, 4, 5, 6, 7, 8]          # 3 role tokens, 5 text tokens, 5 suffix tokens


@pytest.fixture(scope="module")
def rt():
    return T.random_tts(seed=3)


def test_prefill_layout_and_language_rules(rt):
    c = rt.cfg
    prefill, trailing, pad = rt.build_prefill(TEXT, "ryan")
    # role rows + (nothink, think_bos, think_eos, speaker, pad) on the text side's pads / bos + first text token on codec_bos
    assert prefill.shape == (3 + 5 + 1, 64) and trailing.shape == (4 + 1, 64) and pad.shape == (1, 64)
    rows = rt.front(TEXT).float()
    special = rt.front([c.tts_bos_token_id, c.tts_eos_token_id, c.tts_pad_token_id]).float()
    codec = rt.talker.embed_tokens([c.codec_nothink_id, c.codec_think_bos_id, c.codec_think_eos_id, c.speakers["ryan"], c.codec_pad_id, c.codec_bos_id]).float()
    assert torch.allclose(prefill[:3], rows[:3]) and torch.allclose(prefill[3], special[2] + codec[0])
    assert torch.allclose(prefill[7], special[0] + codec[4]) and torch.allclose(prefill[8], rows[3] + codec[5])
    assert torch.allclose(trailing[:4], rows[4:8]) and torch.allclose(trailing[4], special[1])
    # a language adds one row; a dialect speaker switches its dialect on by itself; unknown names fall back to auto
    assert rt.build_prefill(TEXT, "ryan", "english")[0].shape[0] == prefill.shape[0] + 1
    with_dialect = rt.build_prefill(TEXT, "eric")[0]
    assert with_dialect.shape[0] == prefill.shape[0] + 1
    assert torch.allclose(with_dialect[5], special[2] + rt.talker.embed_tokens([c.languages["sichuan_dialect"]]).float()[0])
    assert rt.build_prefill(TEXT, "ryan", "klingon")[0].shape == prefill.shape
    assert c.language_id("auto", "ryan") is None and c.language_id("English", None) == c.languages["english"]
    with pytest.raises(ValueError, match="unknown speaker"):
        rt.build_prefill(TEXT, "nobody")
    with pytest.raises(ValueError, match="shorter"):
        rt.build_prefill(TEXT[:8], "ryan")
    assert rt.voices() == ["eric", "ryan"]


def _dense_hidden(model, rows):
    """Final-norm hidden states of a whole sequence in one cache-free pass through the same modules."""
    from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
    from tensorrt_edge_llm_b200.runtime.runner import ModelRunner
    kv = KVCacheManager(model.cfg, num_pages=8, page_size=16, max_seats=1, max_pages_per_seq=8)
    r = ModelRunner(model, kv)
    meta = r._meta([0], [rows.shape[0]], logits_all=True)
    return model.hidden_states(None, meta, r.cache, inputs_embeds=rows.to(model.cfg.compute_dtype))


def test_greedy_frame_loop_matches_a_cache_free_restatement(rt):
    """Greedy decoding: every frame's codes and every Talker input row are recomputed from scratch (full-sequence passes,
    no KV cache, no runner state) and must agree with what the loop produced."""
    c = rt.cfg
    sp = T.TTSSampling(talker_temperature=0.0, predictor_temperature=0.0, repetition_penalty=1.1, max_audio_length=6)
    codes, reason, tsteps, psteps = rt.generate_codes(TEXT, "ryan", sampling=sp)
    assert codes.shape[1] == c.num_code_groups and 1 <= codes.shape[0] <= 6 and reason in ("eos", "length")
    assert psteps == codes.shape[0] * (c.num_code_groups - 1) and (codes >= 0).all() and (codes < c.codebook_size).all()
    talker, cp = rt.talker.model, rt.predictor.model
    prefill, trailing, pad = rt.build_prefill(TEXT, "ryan")
    seq = prefill
    seen = []
    for f in range(codes.shape[0]):
        h = _dense_hidden(talker, seq)[-1:]
        logits = talker.lm_head(h).float()
        eos = logits[:, c.codec_eos_id].clone()
        logits[:, c.codebook_size:] = float("-inf")
        logits[:, c.codec_eos_id] = eos
        for s in seen:
            logits[0, s] = logits[0, s] / 1.1 if logits[0, s] > 0 else logits[0, s] * 1.1
        c0 = int(logits.argmax(-1))
        assert c0 == int(codes[f, 0])
        seen.append(c0)
        cp_rows = cp.project(torch.cat([h, talker.model.embed_tokens.weight[c0][None]], 0))
        total = talker.model.embed_tokens.weight[c0][None].float()
        for j in range(c.num_code_groups - 1):
            hj = _dense_hidden(cp, cp_rows)[-1:]
            code = int(cp.head_logits(hj, j).argmax(-1))
            assert code == int(codes[f, j + 1]), (f, j)
            row = cp.codec_embeddings[j][code][None]
            total = total + row.float()
            cp_rows = torch.cat([cp_rows, cp.project(row)], 0)
        seq = torch.cat([seq, total + (trailing[f:f + 1] if f < trailing.shape[0] else pad)], 0)
    # sampling: reproducible for one seed, different across seeds, and never a control id
    a = rt.generate_codes(TEXT, "ryan", sampling=T.TTSSampling(max_audio_length=5, seed=7))[0]
    b = rt.generate_codes(TEXT, "ryan", sampling=T.TTSSampling(max_audio_length=5, seed=7))[0]
    d = rt.generate_codes(TEXT, "ryan", sampling=T.TTSSampling(max_audio_length=5, seed=8))[0]
    assert torch.equal(a, b) and (a.shape != d.shape or not torch.equal(a, d)) and (a < c.codebook_size).all()


def test_end_of_stream_stops_the_loop(rt):
    c = rt.cfg
    head = rt.talker.model.lm_head
    saved = head.weight.data.clone()
    greedy = T.TTSSampling(talker_temperature=0.0, predictor_temperature=0.0, max_audio_length=1)
    try:
        rt.generate_codes(TEXT, "ryan", sampling=greedy)                      # one frame: last_hidden is the prefill's last row
        h = rt.talker.model.last_hidden[0]
        head.weight.data[c.codec_eos_id] = 50.0 * torch.sign(h).to(head.weight.dtype)   # end-of-stream now wins the first step
        calls = []
        greedy.max_audio_length = 8
        codes, reason, _, psteps = rt.generate_codes(TEXT, "ryan", sampling=greedy, on_frames=lambda x, final: calls.append((x.shape[0], final)),
                                                     chunk_frames=2)
        assert reason == "eos" and codes.shape == (0, c.num_code_groups) and psteps == 0 and calls == [(0, True)]
        out = rt.generate(TEXT, "ryan", sampling=greedy)
        assert out.frames == 0 and out.waveform.numel() == 0 and out.finish_reason == "eos" and len(out.wav_bytes()) == 44
    finally:
        head.weight.data.copy_(saved)


def test_vocoder_shapes_chunks_and_causality():
    torch.manual_seed(0)
    cfg = Code2WavConfig(codebook_size=20, codebook_dim=8, hidden_size=16, latent_dim=12, num_hidden_layers=2, num_attention_heads=2, intermediate_size=24,
                         sliding_window=3, num_quantizers=3, upsampling_ratios=(2,), upsample_rates=(3, 2), decoder_dim=16)
    m = Code2Wav(cfg).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if not n.endswith("norm.weight"):
                p.copy_(torch.randn(p.shape) * (0.15 if p.dim() > 1 else 0.3))
    assert cfg.samples_per_frame == 12 and cfg.head_dim == 8
    codes = torch.randint(0, 20, (3, 40))
    full = m(codes[None])[0]
    assert full.shape == (40 * 12,) and full.abs().max() <= 1.0 and full.std() > 1e-3 and (full.abs() < 0.999).float().mean() > 0.5
    # causal: changing a later frame leaves every earlier sample as it was
    later = codes.clone()
    later[:, 25] = (later[:, 25] + 1) % 20
    assert torch.equal(m(later[None])[0][: 25 * 12], full[: 25 * 12]) and not torch.equal(m(later[None])[0], full)
    # chunks decoded with the stack's left context reproduce the full decode
    pieces = [m.decode_chunk(codes, s, min(s + 7, 40)) for s in range(0, 40, 7)]
    assert torch.allclose(torch.cat(pieces), full, atol=1e-5)
    short = [m.forward(codes[None, :, max(0, s - 6):min(s + 7, 40)])[0][(s - max(0, s - 6)) * 12:] for s in range(0, 40, 7)]
    assert not torch.allclose(torch.cat(short), full, atol=1e-3)          # too little context does show
    with pytest.raises(ValueError, match="codes per frame"):
        m(codes[None, :2])


def test_generate_streams_chunks_and_round_trips_through_a_directory(rt, tmp_path):
    sp = T.TTSSampling(talker_temperature=0.0, predictor_temperature=0.0, max_audio_length=7)
    whole = rt.generate(TEXT, "ryan", sampling=sp)
    assert whole.frames >= 1 and whole.waveform.shape[0] == whole.frames * rt.code2wav.cfg.samples_per_frame and whole.chunks == 1
    got = []
    streamed = rt.generate(TEXT, "ryan", sampling=sp, chunk_frames=2, on_audio=lambda pcm, sr, final: got.append((len(pcm), sr, final)))
    assert torch.equal(streamed.codes, whole.codes) and torch.allclose(streamed.waveform, whole.waveform, atol=1e-5)
    assert streamed.chunks == (whole.frames + 1) // 2 and got[-1][2] and not any(f for _, _, f in got[:-1])
    assert sum(n for n, _, _ in got) == 2 * whole.waveform.shape[0] and got[0][1] == 24000
    # container: a RIFF file the standard library reads back
    w = wave.open(io.BytesIO(whole.wav_bytes()))
    assert (w.getframerate(), w.getnchannels(), w.getsampwidth(), w.getnframes()) == (24000, 1, 2, whole.waveform.shape[0])
    assert w.readframes(w.getnframes()) == whole.pcm16 == pcm16_bytes(whole.waveform) and wav_file_bytes(b"", 8000)[:4] == b"RIFF"
    # save → load gives the same audio
    d = T.save_tts(str(tmp_path / "tts"), rt)
    again = T.TTS(d).generate(TEXT, "ryan", sampling=sp)
    assert torch.equal(again.codes, whole.codes) and torch.allclose(again.waveform, whole.waveform, atol=1e-6)
    assert T.TTS(d).list_voices() == ["eric", "ryan"] and TTSConfig.from_dict(rt.cfg.to_dict()) == rt.cfg
    with pytest.raises(ValueError, match="tokenizer"):
        rt.generate("plain text")


def test_command_server_routes_and_stage_graph(rt, tmp_path):
    """The same pipeline behind its three front doors: ``trtedge tts``, the HTTP speech routes, a two-stage graph."""
    import json
    from tensorrt_edge_llm_b200.cli import main as trtedge
    d = T.save_tts(str(tmp_path / "tts"), rt)
    greedy = {"talker_temperature": 0.0, "predictor_temperature": 0.0, "max_audio_length": 5}
    want = rt.generate(TEXT, "ryan", sampling=T.TTSSampling.from_dict(greedy))
    # command
    req = tmp_path / "in.json"
    req.write_text(json.dumps({**greedy, "speaker": "ryan", "requests": [{"token_ids": TEXT}, {"token_ids": TEXT, "speaker": "nobody"}]}))
    rc = trtedge(["tts", "--model-dir", d, "--input-file", str(req), "--output-file", str(tmp_path / "out.json"), "--output-audio-dir", str(tmp_path / "wav")])
    rep = json.loads((tmp_path / "out.json").read_text())["responses"]
    assert rc == 1 and rep[0]["frames"] == want.frames and "unknown speaker" in rep[1]["error"]
    assert (tmp_path / "wav" / "request_0.wav").read_bytes() == want.wav_bytes()
    assert trtedge(["tts", "--model-dir", d, "--list-voices"]) == 0
    # HTTP
    from fastapi.testclient import TestClient
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.server.app import create_app
    llm = LLM(tiny_llama_config(num_hidden_layers=1), device="cpu", max_batch_size=1, max_input_len=32, max_kv_cache_capacity=64, page_size=16)
    try:
        c = TestClient(create_app(llm, tts=T.TTS(rt)))
        assert [v["id"] for v in c.get("/v1/voices").json()["data"]] == ["eric", "ryan"]
        r = c.post("/v1/audio/speech", json={"input": TEXT, "voice": "ryan", **greedy})
        assert r.status_code == 200 and r.headers["content-type"] == "audio/wav" and r.content == want.wav_bytes()
        assert r.headers["x-audio-frames"] == str(want.frames)
        r = c.post("/v1/audio/speech", json={"input": TEXT, "voice": "ryan", "response_format": "pcm", "stream": True, "chunk_frames": 2, **greedy})
        assert r.status_code == 200 and len(r.content) == len(want.pcm16)
        got = torch.frombuffer(bytearray(r.content), dtype=torch.int16).int()
        assert (got - torch.frombuffer(bytearray(want.pcm16), dtype=torch.int16).int()).abs().max() <= 1
        for bad in ({"input": TEXT, "voice": "nobody"}, {"input": ""}, {"input": TEXT, "response_format": "mp3"}, {"input": "text needs a tokenizer"}):
            assert c.post("/v1/audio/speech", json=bad).status_code == 400
    finally:
        llm.close()
    # stage graph: talker → vocoder, audio terminal as PCM bytes
    from tensorrt_edge_llm_b200.runtime import multistage as ms
    graph = {"schema_version": 1, "terminals": ["code2wav:audio"], "stages": [
        {"id": "talker", "runner": "tts.talker", "artifact": "tts", "kind": "autoregressive", "config": greedy,
         "inputs": [{"name": "text", "from": "request:text"}, {"name": "voice", "from": "request:voice", "on_missing": "skip"}],
         "emits": [{"id": "codes", "kind": "codec"}]},
        {"id": "code2wav", "runner": "tts.code2wav", "artifact": "tts", "kind": "iterative",
         "inputs": [{"name": "codes", "from": "talker:codes"}], "emits": [{"id": "audio", "kind": "audio", "terminal": True}]}]}
    m = ms.MultiStageRuntime(ms.parse_graph(graph, str(tmp_path)))
    res = m.run([{"text": TEXT, "voice": "ryan"}])
    assert res[0]["ok"] and res[0]["outputs"]["code2wav:audio"] == want.pcm16
    m.close()


def test_code_predictor_head_speculation_is_lossless(rt):
    """Greedy: the speculative pass returns the very codes of the one-code-per-pass loop, for every verify window.  Sampling:
    the second residual code's empirical distribution matches the exact marginal computed by enumeration."""
    c = rt.cfg
    big = T.random_tts(seed=5, groups=7, codebook=24)
    for r in (rt, big):
        greedy = T.TTSSampling(talker_temperature=0.0, predictor_temperature=0.0, max_audio_length=4)
        want = r.generate_codes(TEXT, "ryan", sampling=greedy)
        for n in (2, 3, 8):
            greedy.cp_spec_verify_size = n
            got = r.generate_codes(TEXT, "ryan", sampling=greedy)
            assert torch.equal(got[0], want[0]) and got[1] == want[1], n
            assert got[3] <= want[0].shape[0] * (2 * (r.cfg.num_code_groups - 1))          # passes stay bounded
    with pytest.raises(ValueError, match="2..8"):
        rt.predict_residual_codes_speculative(torch.zeros(1, 64), 3, T.TTSSampling(cp_spec_verify_size=1), 0)
    # make drafts worth accepting: when later heads agree with earlier ones' successors some rounds commit several codes
    sp = T.TTSSampling(predictor_temperature=0.8, predictor_top_k=3, cp_spec_verify_size=3, seed=1)
    rt.generate_codes(TEXT, "ryan", sampling=T.TTSSampling(talker_temperature=0.0, predictor_temperature=0.0, max_audio_length=1))
    h = rt.talker.model.last_hidden.clone()
    cp = rt.predictor.model
    first = 5
    # exact marginal of the second residual code: sum over the first one of P(c1) P(c2 | c1), by dense passes
    x0 = cp.project(torch.cat([h, rt.talker.embed_tokens([first])], 0))
    p1 = rt._distribution(cp.head_logits(_dense_hidden(cp, x0)[-1:], 0), 0.8, 3, 1.0)
    exact = torch.zeros(c.codebook_size)
    for c1 in torch.nonzero(p1).flatten().tolist():
        x1 = torch.cat([x0, cp.project(cp.codec_embeddings[0][c1][None])], 0)
        exact += p1[c1] * rt._distribution(cp.head_logits(_dense_hidden(cp, x1)[-1:], 1), 0.8, 3, 1.0)
    counts = torch.zeros(c.codebook_size)
    trials, multi = 700, 0
    for i in range(trials):
        codes, _, passes = rt.predict_residual_codes_speculative(h, first, sp, 0, generator=torch.Generator().manual_seed(1000 + i))
        counts[codes[1]] += 1
        multi += passes < 1 + (c.num_code_groups - 1)
    tv = 0.5 * (counts / trials - exact).abs().sum()
    assert tv < 0.08, tv
    assert float(counts[exact == 0].sum()) == 0                      # nothing outside the exact support is ever produced


def test_audio_out_graph_hands_the_text_decoder_ids_to_the_talker(rt, tmp_path):
    """Thinker → talker → vocoder: the text decoder's generated ids are wrapped in the speech template and spoken; a
    text-only request leaves the speech stages unloaded."""
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime import multistage as ms
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    T.save_tts(str(tmp_path / "tts"), rt)
    greedy = {"talker_temperature": 0.0, "predictor_temperature": 0.0, "max_audio_length": 4}
    g = ms.parse_graph(ms.audio_out_graph(tts_artifact="tts", talker_config=greedy), str(tmp_path))
    assert ms.validate_graph(g) == ["thinker", "talker", "code2wav"]
    llm = LLM(tiny_llama_config(num_hidden_layers=1, vocab_size=80), device="cpu", max_batch_size=2, max_input_len=32, max_kv_cache_capacity=64, page_size=16)
    try:
        m = ms.MultiStageRuntime(g, stages={"thinker": ms.LLMBackboneStage(g.stage("thinker"), str(tmp_path), llm=llm)})
        res = m.run([{"messages": [3, 4, 5], "sampling": {"max_tokens": 5}, "voice": "ryan"}])[0]
        assert res["ok"], res["error"]
        answer = res["stages"] and llm.generate([[3, 4, 5]], __import__("tensorrt_edge_llm_b200.runtime.runner", fromlist=["SamplingParams"]).SamplingParams(max_tokens=5))[0].token_ids
        want = rt.generate(rt.template_ids(answer), "ryan", sampling=T.TTSSampling.from_dict(greedy))
        assert res["outputs"]["code2wav:audio"] == want.pcm16 and len(want.pcm16) > 0
        m2 = ms.MultiStageRuntime(g, stages={"thinker": ms.LLMBackboneStage(g.stage("thinker"), str(tmp_path), llm=llm)})
        only_text = m2.run([{"messages": [3, 4, 5], "sampling": {"max_tokens": 5}}], want=["thinker:text"])[0]
        assert only_text["ok"] and "talker" not in only_text["stages"] and "talker" not in m2._stages
    finally:
        llm.close()
    assert rt.template_ids([9, 9]) == [1, 2, 3, 9, 9, 4, 5, 6, 7, 8]
    bare = T.TTSConfig()
    with pytest.raises(ValueError, match="role_prefix_ids"):
        T.TTSRuntime.template_ids(type("R", (), {"cfg": bare})(), [1])
