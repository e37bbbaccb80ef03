"""``trtedge tts``: text to speech from a request file (the reference's ``examples/cpp/qwen3_tts_inference.cpp``:
``--input-file --output-file --output-audio-dir``; request file keys as in its guide: top-level ``speaker`` / ``language`` /
``talker_temperature`` / ``talker_top_k`` / ``talker_top_p`` / ``repetition_penalty`` / ``max_audio_length`` defaults and a
``requests`` list whose entries carry ``messages`` (the last assistant message is spoken) or ``text`` / ``token_ids`` and may
override ``speaker`` and ``language``)."""
from __future__ import annotations

import argparse
import json
import os
import time


def _text_of(req: dict):
    if "token_ids" in req:
        return list(req["token_ids"])
    if "text" in req:
        return req["text"]
    msgs = [m for m in req.get("messages", []) if m.get("role") == "assistant"] or req.get("messages", [])
    if not msgs:
        raise ValueError("a request needs messages, text or token_ids")
    content = msgs[-1]["content"]
    return content if isinstance(content, str) else "".join(p.get("text", "") for p in content if isinstance(p, dict))


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge tts")
    p.add_argument("--model-dir", "--talker-engine-dir", dest="model_dir", required=True, help="directory written by save_tts (tts_config.json + weights)")
    p.add_argument("--input-file", "--inputFile", default=None)
    p.add_argument("--text", default=None, help="one request from the command line")
    p.add_argument("--speaker", default=None)
    p.add_argument("--language", default=None)
    p.add_argument("--output-file", "--outputFile", default=None, help="JSON report (frames, seconds, finish reason per request)")
    p.add_argument("--output-audio-dir", "--outputAudioDir", default=None, help="writes request_<i>.wav here")
    p.add_argument("--chunk-frames", type=int, default=0, help="vocode every N frames while the loop is still running (0 = once at the end)")
    p.add_argument("--cp-spec-verify-size", type=int, default=0,
                   help="CodePredictor head speculation: one committed depth plus N-1 drafted depths per pass (0 = off, 2..8)")
    p.add_argument("--device", default="cpu")
    p.add_argument("--list-voices", action="store_true")
    a = p.parse_args(argv)
    from ..runtime.tts import TTS, TTSSampling
    tts = TTS(a.model_dir, device=a.device)
    if a.list_voices:
        print("\n".join(tts.list_voices()))
        return 0
    if a.input_file:
        with open(a.input_file, "r", encoding="utf-8") as f:
            body = json.load(f)
    elif a.text is not None:
        body = {"requests": [{"text": a.text}]}
    else:
        p.error("give --text, --input-file or --list-voices")
    defaults = {k: v for k, v in body.items() if k != "requests"}
    if a.speaker:
        defaults["speaker"] = a.speaker
    if a.language:
        defaults["language"] = a.language
    if a.cp_spec_verify_size:
        if not 2 <= a.cp_spec_verify_size <= 8:
            p.error("--cp-spec-verify-size must be in 2..8 (1 leaves no draft slot)")
        defaults["cp_spec_verify_size"] = a.cp_spec_verify_size
    if a.output_audio_dir:
        os.makedirs(a.output_audio_dir, exist_ok=True)
    report = []
    ok = True
    for i, req in enumerate(body["requests"]):
        merged = {**defaults, **req}
        entry = {"request": i}
        try:
            t0 = time.perf_counter()
            out = tts.generate(_text_of(req), merged.get("speaker"), merged.get("language"), TTSSampling.from_dict(merged), a.chunk_frames)
            dt = time.perf_counter() - t0
            seconds = out.waveform.shape[0] / out.sample_rate
            entry.update(frames=out.frames, audio_seconds=round(seconds, 3), finish_reason=out.finish_reason, wall_seconds=round(dt, 3),
                         real_time_factor=round(dt / seconds, 3) if seconds else None, talker_steps=out.talker_steps, predictor_steps=out.predictor_steps)
            if a.output_audio_dir:
                entry["audio_file"] = os.path.join(a.output_audio_dir, f"request_{i}.wav")
                with open(entry["audio_file"], "wb") as f:
                    f.write(out.wav_bytes())
        except (ValueError, KeyError) as e:
            ok = False
            entry["error"] = f"{type(e).__name__}: {e}"
        report.append(entry)
        print(json.dumps(entry))
    if a.output_file:
        with open(a.output_file, "w", encoding="utf-8") as f:
            json.dump({"responses": report}, f, indent=1)
    return 0 if ok else 1
