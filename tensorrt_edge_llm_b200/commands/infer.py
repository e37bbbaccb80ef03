"""``trtedge infer``: run a request file through a checkpoint and write a predictions file.

Counterpart of the reference's ``examples/cpp/llm_inference.cpp`` with the request format of
``docs/source/user_guide/format/input-format.md`` (``examples/cpp/common/requestFileParser.cpp``): top-level sampling
defaults (``temperature top_p top_k sampling_seed max_generate_length num_logprobs logit_bias guided_decoding
apply_chat_template add_generation_prompt enable_thinking batch_size``) and per-request ``messages`` with overrides
(``sampling_seed logit_bias num_logprobs guided_decoding stop disable_spec_decode``).  ``--dump-profile`` prints the
stage timings and peak device memory."""
from __future__ import annotations

import argparse
import json
import sys
from typing import Any, Dict, List


class RequestFileError(ValueError):
    pass


def _guided(spec):
    from ..runtime.guided import GuidedDecodingParams
    if not spec:
        return None
    modes = [k for k in ("json_object", "json_schema", "regex", "choice", "ebnf", "structural_tag") if spec.get(k) not in (None, False)]
    if len(modes) != 1:
        raise RequestFileError("guided_decoding needs exactly one mode")
    m = modes[0]
    if m == "json_object":
        return GuidedDecodingParams("json_object")
    if m == "json_schema":
        return GuidedDecodingParams("json_schema", json_schema=spec[m] if isinstance(spec[m], dict) else json.loads(spec[m]))
    if m == "regex":
        return GuidedDecodingParams("regex", pattern=str(spec[m]))
    if m == "choice":
        return GuidedDecodingParams("choice", choices=list(spec[m]))
    if m == "ebnf":
        return GuidedDecodingParams("ebnf", grammar=str(spec[m]), jump_forward=bool(spec.get("jump_forward", False)))
    return GuidedDecodingParams("structural_tag", structural_tag=spec[m] if isinstance(spec[m], dict) else json.loads(spec[m]))


def parse_request_file(body: Dict[str, Any]) -> List[Dict[str, Any]]:
    """Validate a request file and resolve the top-level defaults into one flat dict per request."""
    if not isinstance(body, dict) or not isinstance(body.get("requests"), list) or not body["requests"]:
        raise RequestFileError("the file needs a non-empty 'requests' array")
    top_lp = int(body.get("num_logprobs", 0))
    out = []
    for i, r in enumerate(body["requests"]):
        if not isinstance(r, dict) or not isinstance(r.get("messages"), list) or not r["messages"]:
            raise RequestFileError(f"requests[{i}] needs a non-empty 'messages' array")
        for m in r["messages"]:
            if m.get("role") not in ("system", "user", "assistant", "tool") or "content" not in m:
                raise RequestFileError(f"requests[{i}]: every message needs a role and content")
        n_lp = int(r.get("num_logprobs", top_lp))
        if not 0 <= n_lp <= 50:
            raise RequestFileError(f"requests[{i}]: num_logprobs must be in [0, 50]")
        if body.get("context_cache_lookup_policy", "use_cache") not in ("use_cache", "bypass"):
            raise RequestFileError("context_cache_lookup_policy must be use_cache or bypass")
        if body.get("context_cache_commit_policy", "including_generated_tokens") not in ("none", "prefill_state_only", "including_generated_tokens"):
            raise RequestFileError("unknown context_cache_commit_policy")
        bias = r.get("logit_bias", body.get("logit_bias"))
        stop = r.get("stop", [])
        out.append({
            "messages": r["messages"],
            "temperature": float(body.get("temperature", 1.0)), "top_p": float(body.get("top_p", 0.8)), "top_k": int(body.get("top_k", 50)),
            "seed": int(r.get("sampling_seed", body.get("sampling_seed", 42))),
            "max_tokens": int(body.get("max_generate_length", 256)),
            "num_logprobs": n_lp, "logit_bias": {int(k): float(v) for k, v in bias.items()} if bias else None,
            "guided": _guided(r.get("guided_decoding", body.get("guided_decoding"))),
            "stop": [stop] if isinstance(stop, str) else list(stop),
            "apply_chat_template": bool(body.get("apply_chat_template", True)),
            "add_generation_prompt": bool(body.get("add_generation_prompt", True)),
            "enable_thinking": bool(body.get("enable_thinking", False)),
            "disable_spec_decode": bool(r.get("disable_spec_decode", False)), "lora_name": r.get("lora_name"),
            "cache_lookup": body.get("context_cache_lookup_policy", "use_cache") != "bypass",
            "cache_commit": body.get("context_cache_commit_policy", "including_generated_tokens"),
        })
    return out


def _text_of(messages) -> str:
    parts = []
    for m in messages:
        c = m["content"]
        parts.append(c if isinstance(c, str) else "".join(p.get("text", "") for p in c if p.get("type") == "text"))
    return "\n".join(parts)


def _with_media(llm, multimodal, messages, render):
    """Messages with image / audio parts → a prepared multimodal prompt (media files are read from the paths the file names)."""
    import re
    from ..runtime import native as rt
    from ..runtime.multimodal import MultimodalInputs
    from ..server import app as server_app
    server_app._MEDIA_ROOT["path"] = "/"              # an offline command reads the files its own input names
    flat, media = server_app._split_media(messages)
    if not media:
        return render(messages)
    if multimodal is None:
        raise RequestFileError("the request names media but the checkpoint brings no tower this runtime builds")
    if llm.tokenizer is None:
        raise RequestFileError("media requests need a tokenizer")
    req, it = MultimodalInputs(), iter(media)
    for piece in re.split(f"({server_app._IMG}|{server_app._AUD})", render(flat)):
        if piece == server_app._IMG:
            req.image(next(it)[1])
        elif piece == server_app._AUD:
            clip = rt.parse_audio(next(it)[1])
            req.audio(clip.samples, clip.sample_rate)
        elif piece:
            req.text(list(llm.tokenizer.encode(piece)))
    return multimodal.prepare(req)


def run_requests(llm, template, requests: List[Dict[str, Any]], multimodal=None) -> List[Dict[str, Any]]:
    from ..runtime.runner import SamplingParams
    results = []
    for r in requests:
        render = (lambda msgs, r=r: template.apply(msgs, r["add_generation_prompt"], None, r["enable_thinking"])) if r["apply_chat_template"] \
            else _text_of
        prompt = _with_media(llm, multimodal, r["messages"], render)
        sp = SamplingParams(max_tokens=r["max_tokens"], temperature=r["temperature"], top_k=r["top_k"], top_p=r["top_p"], seed=r["seed"],
                            logprobs=r["num_logprobs"] if r["num_logprobs"] > 0 else None, logit_bias=r["logit_bias"], guided=r["guided"],
                            context_cache_lookup=r["cache_lookup"], context_cache_commit=r["cache_commit"],
                            disable_spec_decode=r["disable_spec_decode"])
        o = llm.generate([prompt], sp)[0]
        text = o.text or ""
        reason = o.finish_reason
        cut = min((text.find(s) for s in r["stop"] if s and s in text), default=-1)
        if cut >= 0:
            text, reason = text[:cut], "stop"
        res = {"output_text": text, "output_ids": o.token_ids, "finish_reason": reason, "input_tokens": len(o.prompt_token_ids),
               "output_tokens": len(o.token_ids), "ttft_s": o.ttft_s, "reused_input_tokens": o.reused_input_tokens}
        if o.spec_stats:
            res["spec_decode"] = o.spec_stats
        if o.logprobs:
            res["logprobs"] = [{"token_id": e["token_id"], "logprob": e["logprob"],
                                "top": [{"token_id": t, "logprob": v} for t, v in e["top"]]} for e in o.logprobs]
        results.append(res)
    return results


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge infer")
    p.add_argument("model_dir")
    p.add_argument("--input-file", "--inputFile", required=True)
    p.add_argument("--output-file", "--outputFile", required=True)
    p.add_argument("--max-batch-size", "--maxBatchSize", type=int, default=8)
    p.add_argument("--draft-model", "--draftModel", default=None)
    p.add_argument("--dump-profile", "--dumpProfile", action="store_true")
    p.add_argument("--device", default=None)
    a = p.parse_args(argv)
    from .. import profiling as prof
    from ..chat_template import ChatTemplate
    from ..runtime import native as rt
    from ..runtime.llm import LLM
    try:
        with open(a.input_file, "r", encoding="utf-8") as f:
            requests = parse_request_file(json.load(f))
    except (OSError, json.JSONDecodeError, RequestFileError) as e:
        print(f"bad request file: {e}", file=sys.stderr)
        return 1
    try:
        tok = rt.Tokenizer.load_from_hf(a.model_dir)
    except Exception as e:       # a checkpoint without tokenizer files can still run token-id free text through the fallback below
        print(f"no tokenizer in {a.model_dir}: {e}", file=sys.stderr)
        return 1
    llm = LLM(a.model_dir, device=a.device, max_batch_size=a.max_batch_size, tokenizer=tok, draft_model=a.draft_model)
    prof.set_profiling_enabled(a.dump_profile)
    mon = prof.MemoryMonitor().start() if a.dump_profile else None
    try:
        from ..runtime.multimodal import MultimodalRunner
        results = run_requests(llm, ChatTemplate.load(a.model_dir), requests, MultimodalRunner.from_pretrained(llm, a.model_dir))
    finally:
        peak = mon.stop() if mon else 0
        llm.close()
    with open(a.output_file, "w", encoding="utf-8") as f:
        json.dump({"input_file": a.input_file, "responses": results}, f, indent=1, ensure_ascii=False)
    if a.dump_profile:
        print(prof.timer().format())
        print(f"peak device memory: {peak / 2 ** 20:.1f} MiB")
    return 0
