"""FastAPI application: health, model list, OpenAI chat / completions / responses, Anthropic messages.

Parity: ``tensorrt_edgellm/server/api/routes.py`` (:104 ``/health``, :150 ``/health/ready``, :169
``/v1/models``, :181 ``/v1/chat/completions``, :194 ``/v1/responses``, :238 ``/v1/completions``, :260
``/v1/messages``, :274 ``/v1/messages/count_tokens``), error shapes of ``api/errors.py`` and the
429 / 503 admission behaviour of ``runtime/engine_client.py``.  Audio routes need the speech models
and are not served."""
from __future__ import annotations

import json
import time
import uuid
from typing import Any, Dict, List, Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, StreamingResponse

from ..chat_template import ChatTemplate
from ..runtime.llm import LLM
from ..runtime.runner import SamplingParams
from . import parsing
from .config import ApiConfig
from .engine_client import EngineClient, EngineUnavailable, QueueFull, QueueTimeout


def _error(status: int, message: str, etype: str = "invalid_request_error", code: Optional[str] = None) -> JSONResponse:
    return JSONResponse(status_code=status, content={"error": {"message": message, "type": etype, "param": None, "code": code}})


def _sampling(body: Dict[str, Any], default_max: int = 256) -> SamplingParams:
    max_tokens = body.get("max_completion_tokens") or body.get("max_tokens") or body.get("max_output_tokens") or default_max
    stop_ids = body.get("stop_token_ids") or []
    sp = SamplingParams(temperature=float(body.get("temperature", 0.7) if body.get("temperature") is not None else 0.7),
                        top_k=int(body.get("top_k", 50) or 0), top_p=float(body.get("top_p", 0.9) if body.get("top_p") is not None else 0.9),
                        seed=int(body.get("seed", 42) or 42), ignore_eos=bool(body.get("ignore_eos", False)),
                        stop_token_ids=tuple(int(t) for t in stop_ids))
    sp.max_tokens = int(max_tokens)
    if sp.max_tokens < 1:
        raise ValueError("max_tokens must be at least 1")
    if body.get("max_denoising_steps"):                    # block-diffusion checkpoints: denoise passes per block
        sp.max_denoising_steps = int(body["max_denoising_steps"])
    if body.get("disable_spec_decode"):
        sp.disable_spec_decode = True
    # chat form: logprobs=true + top_logprobs=k; completions form: logprobs=k
    want = body.get("logprobs")
    if isinstance(want, bool):
        sp.logprobs = int(body.get("top_logprobs") or 0) if want else None
    elif want is not None:
        sp.logprobs = int(want)
    if sp.logprobs is not None and not 0 <= sp.logprobs <= 50:
        raise ValueError("top_logprobs must be in 0..50")
    bias = body.get("logit_bias")
    if bias:
        if not isinstance(bias, dict):
            raise ValueError("logit_bias must map token ids to biases")
        sp.logit_bias = {int(k): float(v) for k, v in bias.items()}
    return sp


def _guided(body: Dict[str, Any]):
    """OpenAI ``response_format`` and the ``guided_choice`` / ``guided_regex`` / ``guided_json`` extensions → matcher parameters."""
    from ..runtime.guided import GuidedDecodingParams
    if body.get("guided_choice"):
        return GuidedDecodingParams("choice", choices=list(body["guided_choice"]))
    if body.get("guided_regex"):
        return GuidedDecodingParams("regex", pattern=str(body["guided_regex"]))
    if body.get("guided_json"):
        return GuidedDecodingParams("json_schema", json_schema=body["guided_json"])
    if body.get("guided_grammar"):
        return GuidedDecodingParams("ebnf", grammar=str(body["guided_grammar"]))
    if body.get("structural_tag"):
        st = body["structural_tag"]
        return GuidedDecodingParams("structural_tag", structural_tag=json.loads(st) if isinstance(st, str) else st)
    rf = body.get("response_format") or {}
    if rf.get("type") == "json_object":
        return GuidedDecodingParams("json_object")
    if rf.get("type") == "structural_tag":
        return GuidedDecodingParams("structural_tag", structural_tag={k: rf[k] for k in ("structures", "triggers") if k in rf})
    if rf.get("type") == "json_schema":
        schema = (rf.get("json_schema") or {}).get("schema")
        return GuidedDecodingParams("json_schema", json_schema=schema)
    return None


_IMG, _AUD = "\x00IMG\x00", "\x00AUD\x00"


# Directory under which requests may name local media files ("" = none: only data: URIs are read).  Set by `create_app`
# from `ApiConfig.allowed_local_media_path` (``--allowed-local-media-path`` in the reference's server as well).
_MEDIA_ROOT = {"path": ""}


def _media_bytes(ref: str) -> bytes:
    """``data:…;base64,…`` URI, or a ``file://`` URI / local path under the allowed media directory → bytes (no network
    fetches; without an allowed directory a request cannot make the server read its files)."""
    import base64
    import os
    if ref.startswith("data:"):
        return base64.b64decode(ref.split(",", 1)[1])
    if ref.startswith(("http://", "https://")):
        raise ValueError("remote media URLs are not fetched; send a data: URI")
    root = _MEDIA_ROOT["path"]
    if not root:
        raise ValueError("local media paths are disabled on this server (start it with --allowed-local-media-path); send a data: URI")
    path = os.path.realpath(ref[7:] if ref.startswith("file://") else ref)
    root = os.path.realpath(root)
    if os.path.commonpath([path, root]) != root:
        raise ValueError("media path is outside the allowed directory")
    with open(path, "rb") as f:
        return f.read()


def _split_media(messages):
    """Content parts → plain-text messages with markers where media sits, plus the media in order of appearance."""
    media, flat = [], []
    for m in messages:
        c = m.get("content")
        if not isinstance(c, list):
            flat.append(m)
            continue
        text = ""
        for part in c:
            kind = part.get("type")
            if kind == "text":
                text += part.get("text", "")
            elif kind in ("image", "image_url"):
                src = part.get("image") or (part.get("image_url") or {}).get("url")
                source = part.get("source")
                if src is None and isinstance(source, dict):            # Anthropic block: {"type": "base64", "media_type", "data"} or a URL
                    src = ("data:" + str(source.get("media_type", "image/png")) + ";base64," + str(source.get("data", ""))
                           if source.get("type") == "base64" else source.get("url"))
                media.append(("image", _media_bytes(str(src))))
                text += _IMG
            elif kind == "video":                                   # a clip as a list of frame images (Qwen-VL request format)
                frames = part.get("video")
                if not isinstance(frames, list) or not frames:
                    raise ValueError("a video part needs a list of frame images (data: URIs or allowed local paths)")
                media.append(("image", [_media_bytes(str(f)) for f in frames]))
                text += _IMG
            elif kind in ("audio", "input_audio", "audio_url"):
                src = part.get("audio") or (part.get("audio_url") or {}).get("url")
                if src is None and isinstance(part.get("input_audio"), dict):
                    src = "data:audio/wav;base64," + part["input_audio"]["data"]
                media.append(("audio", _media_bytes(str(src))))
                text += _AUD
            else:
                raise ValueError(f"unsupported content part {kind!r}")
        flat.append({**m, "content": text})
    return flat, media


def _truncate_at_stop(text: str, stops) -> (str, bool):
    if isinstance(stops, str):
        stops = [stops]
    cut = min((text.find(s) for s in (stops or []) if s and s in text), default=-1)
    return (text[:cut], True) if cut >= 0 else (text, False)


def create_app(llm: LLM, api: Optional[ApiConfig] = None, chat_template: Optional[ChatTemplate] = None,
               model_name: str = "", multimodal=None, tts=None) -> FastAPI:
    """``tts``: a ``runtime.tts.TTS`` (or ``TTSRuntime``); ``/v1/audio/speech`` and ``/v1/voices`` are answered by it.
    ``multimodal``: a ``runtime.multimodal.MultimodalRunner`` over ``llm``; chat requests whose messages carry image or
    audio parts are then answered through it: on the request engine next to all other requests when in-flight batching is on,
    otherwise one at a time on the static path."""
    api = api or ApiConfig()
    _MEDIA_ROOT["path"] = api.allowed_local_media_path
    client = EngineClient(llm, api.max_queued_requests, api.queue_timeout)
    template = chat_template or ChatTemplate()
    name = api.served_model_name or model_name or "model"
    reasoning = parsing.resolve_reasoning_parser(api.reasoning_parser, getattr(template, "source", ""))
    app = FastAPI(title="tensorrt_edge_llm_b200", version="1")
    app.state.client, app.state.started = client, time.time()

    @app.middleware("http")
    async def auth(request: Request, call_next):
        if api.api_key and request.url.path.startswith("/v1"):
            got = request.headers.get("authorization", "")
            key = request.headers.get("x-api-key", "")
            if got != f"Bearer {api.api_key}" and key != api.api_key:
                return _error(401, "invalid API key", "authentication_error")
        return await call_next(request)

    def encode(text: str) -> List[int]:
        if llm.tokenizer is None:
            raise ValueError("this server has no tokenizer: send token ids (prompt as a list of integers)")
        return list(llm.tokenizer.encode(text))

    def decode(ids: List[int]) -> str:
        if llm.tokenizer is None:
            return ""
        t = llm.tokenizer.decode(ids)
        return t.decode("utf-8", "replace") if isinstance(t, (bytes, bytearray)) else t

    def check_len(ids: List[int]) -> Optional[JSONResponse]:
        if not ids:
            return _error(400, "empty prompt")
        if len(ids) > llm.max_input_len:
            return _error(400, f"prompt has {len(ids)} tokens, the server accepts {llm.max_input_len}", code="context_length_exceeded")
        return None

    async def run(ids: List[int], sp: SamplingParams, priority: int = 0):
        try:
            return await client.generate(ids, sp, priority), None
        except QueueFull as e:
            return None, _error(429, f"server is at capacity: {e}", "rate_limit_error")
        except (QueueTimeout, EngineUnavailable) as e:
            return None, _error(503, f"engine unavailable: {e}", "service_unavailable")
        except (ValueError, RuntimeError) as e:
            return None, _error(400, str(e))

    def sse(gen):
        return StreamingResponse(gen, media_type="text/event-stream", headers={"Cache-Control": "no-cache", "X-Accel-Buffering": "no"})

    # ---- health / models -----------------------------------------------------------------------------------
    def _capabilities():
        spec = llm.spec_decoder
        audio = multimodal is not None and multimodal.audio is not None
        vision = multimodal is not None and multimodal.vision is not None
        return {"chat": True, "transcription": audio, "speech": False,
                "input_modalities": ["text"] + (["image"] if vision else []) + (["audio"] if audio else []), "output_modalities": ["text"],
                "max_model_len": llm.kv.max_pages_per_seq * llm.kv.page_size, "max_input_len": llm.max_input_len,
                "max_batch_size": llm.max_batch_size, "max_num_seqs": llm.max_batch_size, "kv_cache_dtype": str(llm.kv.pool.dtype).replace("torch.", ""),
                "speculative_decoding": spec is not None or llm.diffusion_decoder is not None,
                "speculative_method": getattr(spec, "name", "eagle3" if spec is not None else ("block_diffusion" if llm.diffusion_decoder is not None else None)),
                "context_reuse": bool(getattr(getattr(llm, "session", None), "prefix", None) is not None), "in_flight_batching": llm.engine is not None}

    def _engine_report():
        """Engine status, scheduling counters and context-cache counters of the native request engine (``None`` without one)."""
        if llm.engine is None:
            return None, None, None
        st = llm.engine.status()
        engine = {"serving": bool(st.available), "unavailable_reason": st.unavailable_reason, "queued": int(st.queued), "resident": int(st.resident)}
        scheduling, cache = llm.get_scheduling_metrics(), llm.get_context_cache_counters()
        return engine, scheduling, cache

    @app.get("/health")
    async def health():
        """Liveness with the engine's counters (``tensorrt_edgellm/server/api/routes.py:104``): 503 once the engine refuses work."""
        running, waiting = client.admission.depth
        engine, scheduling, cache = _engine_report()
        healthy = engine is None or engine["serving"]
        body = {"status": "healthy" if healthy else "unhealthy", "model": name, "uptime_s": round(time.time() - app.state.started, 1),
                "active_requests": running, "queued_requests": waiting, "running": running, "queued": waiting,
                "scheduling": scheduling, "context_cache": cache, "engine": engine, "capabilities": _capabilities()}
        if not healthy:
            body["reason"] = engine["unavailable_reason"]
            return JSONResponse(status_code=503, content=body)
        return body

    @app.get("/health/ready")
    async def ready():
        ok, why = client.ready()
        running, waiting = client.admission.depth
        if not ok:
            return JSONResponse(status_code=503, content={"status": "unavailable", "reason": why or "not ready", "active_requests": running,
                                                          "queued_requests": waiting, "error": {"message": why or "not ready", "type": "service_unavailable"}})
        return {"status": "ready", "active_requests": running, "queued_requests": waiting}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": name, "object": "model", "created": int(app.state.started), "owned_by": "local",
                                            "max_model_len": llm.max_input_len}]}

    def _media_request(prompt, media):
        """Rendered prompt with media markers → text pieces and decoded media in order."""
        import re
        from ..runtime import native as rt
        from ..runtime.multimodal import MultimodalInputs
        req, it = MultimodalInputs(), iter(media)
        for piece in re.split(f"({_IMG}|{_AUD})", prompt):
            if piece == _IMG:
                req.image(next(it)[1])
            elif piece == _AUD:
                clip = rt.parse_audio(next(it)[1])
                req.audio(clip.samples, clip.sample_rate)
            elif piece:
                req.text(encode(piece))
        return req

    async def _multimodal_chat(body, messages, media, sp):
        import asyncio
        prompt = template.apply(messages, True, None, bool((body.get("chat_template_kwargs") or {}).get("enable_thinking", True)))
        req = _media_request(prompt, media)

        def work():
            client.admission.acquire()
            try:
                if llm.engine is not None:             # the request engine batches it with everything else in flight
                    return multimodal.generate(req, max_tokens=sp.max_tokens)
                with client._lock:
                    return multimodal.generate(req, max_tokens=sp.max_tokens)
            finally:
                client.admission.release()
        toks = await asyncio.get_running_loop().run_in_executor(None, work)
        n_in = sum(len(p) if k == "text" else 0 for k, p in req.pieces)
        return {"id": f"chatcmpl-{uuid.uuid4().hex[:24]}", "object": "chat.completion", "created": int(time.time()), "model": name,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": decode(toks)}, "finish_reason": "length",
                             "token_ids": toks}],
                "usage": {"prompt_tokens": n_in, "completion_tokens": len(toks), "total_tokens": n_in + len(toks)}}

    # ---- audio ------------------------------------------------------------------------------------------------
    @app.post("/v1/audio/transcriptions")
    async def audio_transcriptions(request: Request):
        """OpenAI transcription route (``tensorrt_edgellm/server/api/routes.py:283``): a multipart form with the audio ``file``
        (WAV) and optional ``prompt``, ``language``, ``response_format`` (json | text), ``temperature``.  The clip goes through
        the audio encoder and the language model answers an instruction to transcribe it."""
        import asyncio
        from ..runtime import native as rt
        from ..runtime.multimodal import MultimodalInputs
        if multimodal is None or multimodal.audio is None:
            return _error(400, "the loaded model has no audio encoder: transcription is not available", code="model_capability")
        try:
            form = await request.form()
            upload = form.get("file")
            if upload is None or not hasattr(upload, "read"):
                raise ValueError("the form needs an audio 'file'")
            data = await upload.read()
            fmt = str(form.get("response_format", "json") or "json")
            if fmt not in ("json", "text"):
                raise ValueError("response_format must be json or text")
            clip = rt.parse_audio(data)
            hint, language = str(form.get("prompt", "") or ""), str(form.get("language", "") or "")
            ask = "Transcribe the audio" + (f" (language: {language})" if language else "") + "." + (f" {hint}" if hint else "")
            prompt = template.apply([{"role": "user", "content": _AUD + ask}], True, None, False)
            # one clip: text before the marker, the clip, text after it
            before, _, after = prompt.partition(_AUD)
            req = MultimodalInputs()
            if before:
                req.text(encode(before))
            req.audio(clip.samples, clip.sample_rate)
            if after:
                req.text(encode(after))
            limit = int(form.get("max_tokens", 256) or 256)
        except (ValueError, RuntimeError, KeyError) as e:
            return _error(400, f"bad request: {e}")

        def work():
            client.admission.acquire()
            try:
                if llm.engine is not None:
                    return multimodal.generate(req, max_tokens=limit)
                with client._lock:
                    return multimodal.generate(req, max_tokens=limit)
            finally:
                client.admission.release()
        toks = await asyncio.get_running_loop().run_in_executor(None, work)
        eos = llm.cfg.eos_token_id
        eos = set(eos if isinstance(eos, (list, tuple)) else [eos]) - {None}
        cut = next((i for i, t in enumerate(toks) if t in eos), len(toks))
        text = decode(toks[:cut]).strip()
        if fmt == "text":
            from fastapi.responses import PlainTextResponse
            return PlainTextResponse(text)
        return {"text": text, "usage": {"type": "tokens", "output_tokens": cut, "seconds": round(len(clip.samples) / max(clip.sample_rate, 1), 3)}}

    @app.get("/v1/voices")
    async def voices():
        names = list(llm.list_voices()) + (list(speech.voices()) if speech is not None else [])
        return {"object": "list", "data": [{"id": v, "object": "voice"} for v in names]}

    speech = getattr(tts, "runtime", tts)                   # the frame loop serves one request at a time
    speech_lock = __import__("threading").Lock()

    @app.post("/v1/audio/speech")
    async def audio_speech(request: Request):
        """OpenAI speech route: ``input`` (text, or templated token ids), ``voice``, ``response_format`` ``wav`` | ``pcm``;
        ``stream: true`` sends 16-bit PCM chunk by chunk while later frames are still being generated.  Extra keys:
        ``language`` and the sampling keys of the reference's request file (``talker_temperature``, ``talker_top_k``,
        ``talker_top_p``, ``repetition_penalty``, ``max_audio_length``, ``seed``)."""
        if speech is None:
            return _error(400, "the loaded model has no speech synthesis stage", code="model_capability")
        from ..runtime.tts import TTSSampling
        try:
            body = await request.json()
            text = body["input"]
            if not (isinstance(text, str) and text) and not (isinstance(text, list) and text and all(isinstance(t, int) for t in text)):
                raise ValueError("input must be a non-empty string or a list of token ids")
            fmt = body.get("response_format", "wav")
            if fmt not in ("wav", "pcm"):
                raise ValueError("response_format must be wav or pcm")
            voice, language = body.get("voice") or None, body.get("language") or None
            if voice and voice.lower() not in speech.voices():
                raise ValueError(f"unknown voice {voice!r}; available: {speech.voices()}")
            sampling = TTSSampling.from_dict(body)
            ids = speech.tokenize(text) if isinstance(text, str) else list(text)
            speech.build_prefill(ids, voice, language)           # layout errors surface as 400s, before any audio is promised
        except (KeyError, ValueError, TypeError) as e:
            return _error(400, f"bad request: {e}")
        import asyncio
        import queue as queue_mod
        from fastapi.responses import Response
        loop = asyncio.get_running_loop()
        if not body.get("stream"):
            def run():
                with speech_lock:
                    return speech.generate(ids, voice, language, sampling)
            out = await loop.run_in_executor(None, run)
            data = out.wav_bytes() if fmt == "wav" else out.pcm16
            return Response(content=data, media_type="audio/wav" if fmt == "wav" else "audio/pcm",
                            headers={"x-audio-frames": str(out.frames), "x-sample-rate": str(out.sample_rate), "x-finish-reason": out.finish_reason})
        chunks: "queue_mod.Queue" = queue_mod.Queue()

        def produce():
            try:
                with speech_lock:
                    speech.generate(ids, voice, language, sampling, chunk_frames=int(body.get("chunk_frames", 12)),
                                    on_audio=lambda pcm, sr, final: chunks.put(pcm))
            except Exception as e:          # the stream has begun: end it, the error goes to the log
                print(f"speech generation failed: {type(e).__name__}: {e}")
            finally:
                chunks.put(None)

        loop.run_in_executor(None, produce)

        async def body_iter():
            while True:
                piece = await loop.run_in_executor(None, chunks.get)
                if piece is None:
                    return
                if piece:
                    yield piece

        return StreamingResponse(body_iter(), media_type="audio/pcm", headers={"x-sample-rate": str(speech.code2wav.cfg.sample_rate)})

    # ---- OpenAI chat completions ---------------------------------------------------------------------------
    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        try:
            body = await request.json()
            messages = body["messages"]
            if not isinstance(messages, list) or not messages:
                raise ValueError("messages must be a non-empty list")
            sp = _sampling(body)
            tool_cfg = parsing.validate_tool_request(body)
            messages, media = _split_media(messages)
            if media:
                if multimodal is None:
                    raise ValueError("this server has no multimodal runner: send text-only messages")
                if llm.engine is None:
                    return await _multimodal_chat(body, messages, media, sp)
            prompt = template.apply(messages, True, body.get("tools"), bool((body.get("chat_template_kwargs") or {}).get("enable_thinking", True)))
            if media:
                # in-flight batching: encode the media now, then the prepared prompt takes the same road as a text prompt
                # (streaming, tools, reasoning, log-probabilities, priorities)
                import asyncio
                ids = await asyncio.get_running_loop().run_in_executor(None, multimodal.prepare, _media_request(prompt, media))
            else:
                ids = encode(prompt)
        except (KeyError, ValueError, TypeError, RuntimeError, json.JSONDecodeError) as e:
            return _error(400, f"bad request: {e}")
        want_parse = reasoning is not None or tool_cfg.parse_output
        bad = check_len(ids)
        if bad:
            return bad
        rid, created = f"chatcmpl-{uuid.uuid4().hex[:24]}", int(time.time())
        priority = int(body.get("priority", 0) or 0)
        try:
            guided = _guided(body)
        except ValueError as e:
            return _error(400, f"bad request: {e}")
        if guided is not None:
            try:
                out = await client.generate_guided(ids, sp, guided)
            except (QueueFull, QueueTimeout, EngineUnavailable) as e:
                return _error(503 if not isinstance(e, QueueFull) else 429, str(e), "service_unavailable")
            except ValueError as e:
                return _error(400, str(e))
        elif body.get("stream"):
            async def events():
                head = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": name}
                yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]}) + "\n\n"
                n_out = 0
                sp_parser = parsing.StreamingAssistantOutputParser(tool_cfg, reasoning) if want_parse else None

                def chunks(events):
                    for e in events:
                        if e["type"] == "content":
                            delta = {"content": e["text"]}
                        elif e["type"] == "reasoning":
                            delta = {"reasoning_content": e["text"]}
                        else:
                            delta = {"tool_calls": [e["call"].to_openai(e["index"])]}
                        yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": delta, "finish_reason": None}]}) + "\n\n"
                try:
                    async for d in client.stream(ids, sp, priority):
                        n_out += len(d.token_ids)
                        if d.text and sp_parser is not None:
                            for c in chunks(sp_parser.feed(d.text)):
                                yield c
                        elif d.text:
                            yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {"content": d.text}, "finish_reason": None}]}) + "\n\n"
                        if d.finished:
                            fin = d.finish_reason or "stop"
                            if sp_parser is not None:
                                for c in chunks(sp_parser.flush()):
                                    yield c
                                if sp_parser.saw_tool_call and fin == "stop":
                                    fin = "tool_calls"
                            yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {}, "finish_reason": fin}],
                                                         "usage": {"prompt_tokens": len(ids), "completion_tokens": n_out, "total_tokens": len(ids) + n_out}}) + "\n\n"
                except (QueueFull, QueueTimeout, EngineUnavailable) as e:
                    yield "data: " + json.dumps({"error": {"message": str(e), "type": "service_unavailable"}}) + "\n\n"
                yield "data: [DONE]\n\n"
            return sse(events())
        else:
            out, err = await run(ids, sp, priority)
            if err:
                return err
        text, stopped = _truncate_at_stop(out.text if out.text is not None else decode(out.token_ids), body.get("stop"))
        message: Dict[str, Any] = {"role": "assistant", "content": text}
        finish = "stop" if stopped else out.finish_reason
        choice_extra: Dict[str, Any] = {}
        if out.logprobs:
            choice_extra["logprobs"] = {"content": [
                {"token": decode([e["token_id"]]), "token_id": e["token_id"], "logprob": e["logprob"],
                 "top_logprobs": [{"token": decode([t]), "token_id": t, "logprob": v} for t, v in e["top"]]} for e in out.logprobs]}
        if want_parse:
            parsed = parsing.parse_assistant_output(text, tool_cfg, reasoning)
            message["content"] = parsed.content or (None if parsed.tool_calls else "")
            if parsed.reasoning:
                message["reasoning_content"] = parsed.reasoning
            if parsed.tool_calls:
                message["tool_calls"] = [c.to_openai() for c in parsed.tool_calls]
                if finish == "stop":
                    finish = "tool_calls"
        return {"id": rid, "object": "chat.completion", "created": created, "model": name,
                "choices": [{"index": 0, "message": message, "finish_reason": finish, "token_ids": out.token_ids, **choice_extra}],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out.token_ids), "total_tokens": len(ids) + len(out.token_ids)}}

    # ---- OpenAI completions --------------------------------------------------------------------------------
    @app.post("/v1/completions")
    async def completions(request: Request):
        try:
            body = await request.json()
            prompt = body["prompt"]
            ids = [int(t) for t in prompt] if isinstance(prompt, list) and prompt and not isinstance(prompt[0], str) else encode(
                prompt if isinstance(prompt, str) else prompt[0])
            sp = _sampling(body, default_max=16)
        except (KeyError, ValueError, TypeError, IndexError, json.JSONDecodeError) as e:
            return _error(400, f"bad request: {e}")
        bad = check_len(ids)
        if bad:
            return bad
        rid, created = f"cmpl-{uuid.uuid4().hex[:24]}", int(time.time())
        if body.get("stream"):
            async def events():
                async for d in client.stream(ids, sp):
                    yield "data: " + json.dumps({"id": rid, "object": "text_completion", "created": created, "model": name,
                                                 "choices": [{"index": 0, "text": d.text, "token_ids": d.token_ids,
                                                              "finish_reason": d.finish_reason if d.finished else None}]}) + "\n\n"
                yield "data: [DONE]\n\n"
            return sse(events())
        out, err = await run(ids, sp)
        if err:
            return err
        text, stopped = _truncate_at_stop(out.text if out.text is not None else decode(out.token_ids), body.get("stop"))
        extra: Dict[str, Any] = {}
        if out.logprobs:
            extra["logprobs"] = {"tokens": [decode([e["token_id"]]) for e in out.logprobs], "token_ids": [e["token_id"] for e in out.logprobs],
                                 "token_logprobs": [e["logprob"] for e in out.logprobs],
                                 "top_logprobs": [{str(t): v for t, v in e["top"]} for e in out.logprobs]}
        return {"id": rid, "object": "text_completion", "created": created, "model": name,
                "choices": [{"index": 0, "text": text, "token_ids": out.token_ids, "finish_reason": "stop" if stopped else out.finish_reason, **extra}],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out.token_ids), "total_tokens": len(ids) + len(out.token_ids)}}

    # ---- OpenAI responses (text in, text out) ---------------------------------------------------------------
    async def prompt_from_messages(messages):
        """Token ids of rendered messages, or a prepared multimodal prompt when they carry image / audio parts."""
        msgs, media = _split_media(messages)
        text = template.apply(msgs, True)
        if not media:
            return encode(text)
        if multimodal is None or llm.engine is None:
            raise ValueError("image / audio parts need a server with an encoder for them and in-flight batching")
        import asyncio
        return await asyncio.get_running_loop().run_in_executor(None, multimodal.prepare, _media_request(text, media))

    def _responses_messages(body):
        """OpenAI Responses input → chat messages (``input_text`` / ``output_text`` parts are text, ``input_image`` an image)."""
        inp = body["input"]
        if isinstance(inp, str):
            messages = [{"role": "user", "content": inp}]
        else:
            messages = []
            for m in inp:
                c = m.get("content", "")
                if isinstance(c, list):
                    parts = []
                    for part in c:
                        kind = part.get("type")
                        if kind in ("input_text", "output_text", "text"):
                            parts.append({"type": "text", "text": part.get("text", "")})
                        elif kind == "input_image":
                            parts.append({"type": "image_url", "image_url": {"url": part.get("image_url")}})
                        elif kind == "input_audio":
                            parts.append(part)
                        else:
                            raise ValueError(f"unsupported input part {kind!r}")
                    c = parts if any(p["type"] != "text" for p in parts) else "".join(p["text"] for p in parts)
                messages.append({"role": m.get("role", "user"), "content": c})
        if body.get("instructions"):
            messages.insert(0, {"role": "system", "content": body["instructions"]})
        return messages

    @app.post("/v1/responses")
    async def responses(request: Request):
        try:
            body = await request.json()
            sp = _sampling(body)
            if body.get("max_output_tokens"):
                sp.max_tokens = int(body["max_output_tokens"])
            ids = await prompt_from_messages(_responses_messages(body))
        except (KeyError, ValueError, TypeError, AttributeError, RuntimeError, json.JSONDecodeError) as e:
            return _error(400, f"bad request: {e}")
        bad = check_len(ids)
        if bad:
            return bad
        rid, mid = f"resp_{uuid.uuid4().hex[:24]}", f"msg_{uuid.uuid4().hex[:24]}"

        def envelope(status, text, n_out):
            return {"id": rid, "object": "response", "created_at": int(time.time()), "status": status, "model": name,
                    "output": [] if status == "in_progress" else [
                        {"type": "message", "id": mid, "role": "assistant", "status": "completed",
                         "content": [{"type": "output_text", "text": text, "annotations": []}]}],
                    "output_text": text,
                    "usage": {"input_tokens": len(ids), "output_tokens": n_out, "total_tokens": len(ids) + n_out}}
        if body.get("stream"):
            async def events():
                seq = 0

                def ev(kind, data):
                    nonlocal seq
                    seq += 1
                    return f"event: {kind}\ndata: {json.dumps({'type': kind, 'sequence_number': seq, **data})}\n\n"
                yield ev("response.created", {"response": envelope("in_progress", "", 0)})
                yield ev("response.output_item.added", {"output_index": 0, "item": {"type": "message", "id": mid, "role": "assistant",
                                                                                   "status": "in_progress", "content": []}})
                text, n_out = "", 0
                async for d in client.stream(ids, sp):
                    n_out += len(d.token_ids)
                    if d.text:
                        text += d.text
                        yield ev("response.output_text.delta", {"item_id": mid, "output_index": 0, "content_index": 0, "delta": d.text})
                yield ev("response.output_text.done", {"item_id": mid, "output_index": 0, "content_index": 0, "text": text})
                yield ev("response.completed", {"response": envelope("completed", text, n_out)})
            return sse(events())
        out, err = await run(ids, sp)
        if err:
            return err
        text = out.text if out.text is not None else decode(out.token_ids)
        return envelope("completed", text, len(out.token_ids))

    # ---- Anthropic messages --------------------------------------------------------------------------------
    def anthropic_messages(body: Dict[str, Any]) -> List[Dict[str, Any]]:
        msgs: List[Dict[str, Any]] = []
        system = body.get("system")
        if system:
            msgs.append({"role": "system", "content": system if isinstance(system, str) else
                         "".join(b.get("text", "") for b in system if isinstance(b, dict))})
        for m in body["messages"]:
            c = m.get("content", "")
            if not isinstance(c, str):
                if any(isinstance(b, dict) and b.get("type") == "image" for b in c):
                    msgs.append({"role": m["role"], "content": [b for b in c if isinstance(b, dict) and b.get("type") in ("text", "image")]})
                    continue
                c = "".join(b.get("text", "") for b in c if isinstance(b, dict) and b.get("type") == "text")
            msgs.append({"role": m["role"], "content": c})
        return msgs

    async def anthropic_prompt(body):
        """Prompt of an Anthropic request: token ids, or a prepared multimodal prompt when image blocks are present."""
        return await prompt_from_messages(anthropic_messages(body))

    @app.post("/v1/messages")
    async def messages(request: Request):
        try:
            body = await request.json()
            if "max_tokens" not in body:
                raise ValueError("max_tokens is required")
            sp = _sampling(body)
            sp.stop_token_ids = tuple(sp.stop_token_ids)
            ids = await anthropic_prompt(body)
        except (KeyError, ValueError, TypeError, RuntimeError, json.JSONDecodeError) as e:
            return JSONResponse(status_code=400, content={"type": "error", "error": {"type": "invalid_request_error", "message": str(e)}})
        bad = check_len(ids)
        if bad:
            return bad
        mid = f"msg_{uuid.uuid4().hex[:24]}"
        if body.get("stream"):
            async def events():
                def ev(kind, data):
                    return f"event: {kind}\ndata: {json.dumps({'type': kind, **data})}\n\n"
                yield ev("message_start", {"message": {"id": mid, "type": "message", "role": "assistant", "model": name, "content": [],
                                                       "stop_reason": None, "usage": {"input_tokens": len(ids), "output_tokens": 0}}})
                yield ev("content_block_start", {"index": 0, "content_block": {"type": "text", "text": ""}})
                n_out, reason = 0, "end_turn"
                async for d in client.stream(ids, sp):
                    n_out += len(d.token_ids)
                    if d.text:
                        yield ev("content_block_delta", {"index": 0, "delta": {"type": "text_delta", "text": d.text}})
                    if d.finished:
                        reason = "max_tokens" if d.finish_reason == "length" else "end_turn"
                yield ev("content_block_stop", {"index": 0})
                yield ev("message_delta", {"delta": {"stop_reason": reason, "stop_sequence": None}, "usage": {"output_tokens": n_out}})
                yield ev("message_stop", {})
            return sse(events())
        out, err = await run(ids, sp)
        if err:
            return err
        text, stopped = _truncate_at_stop(out.text if out.text is not None else decode(out.token_ids), body.get("stop_sequences"))
        return {"id": mid, "type": "message", "role": "assistant", "model": name, "content": [{"type": "text", "text": text}],
                "stop_reason": "stop_sequence" if stopped else ("max_tokens" if out.finish_reason == "length" else "end_turn"),
                "stop_sequence": None, "usage": {"input_tokens": len(ids), "output_tokens": len(out.token_ids)}}

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(request: Request):
        try:
            body = await request.json()
            return {"input_tokens": len(await anthropic_prompt(body))}
        except (KeyError, ValueError, TypeError, json.JSONDecodeError) as e:
            return JSONResponse(status_code=400, content={"type": "error", "error": {"type": "invalid_request_error", "message": str(e)}})

    return app
