"""``trtedge stream``: run a request file and print the answers while they are generated.

Counterpart of the reference's ``examples/cpp/llm_stream`` example: the requests of the file (format of ``trtedge infer``)
go through the native runtime façade (``csrc/runtime/inference_runtime.cpp``: chat template, tokeniser, request engine with
in-flight batching, incremental detokenisation, stop sequences), and every piece of text is written as soon as it is
complete UTF-8 — one JSON line per event (``{"request": i, "text": "...", "tokens": [...]}``, then a closing line per
request with its finish reason and timings).  ``--plain`` prints the raw text of a single-request file instead."""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge stream")
    p.add_argument("model_dir")
    p.add_argument("--input-file", "--inputFile", required=True, help="request file (see `trtedge infer`)")
    p.add_argument("--max-batch-size", type=int, default=0, help="seats of the request engine (default: the file's request count, at most 8)")
    p.add_argument("--max-input-len", type=int, default=4096)
    p.add_argument("--max-kv-cache-capacity", type=int, default=8192)
    p.add_argument("--plain", action="store_true", help="print only the text (files with one request)")
    p.add_argument("--device", default=None)
    a = p.parse_args(argv)
    from ..runtime import native as rt
    from ..runtime.llm import LLM
    from .infer import RequestFileError, parse_request_file
    try:
        with open(a.input_file, "r", encoding="utf-8") as f:
            reqs = parse_request_file(json.load(f))
    except (OSError, json.JSONDecodeError, RequestFileError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if a.plain and len(reqs) != 1:
        print("error: --plain needs a file with exactly one request", file=sys.stderr)
        return 2
    first = reqs[0]
    for r in reqs[1:]:                     # the façade takes one sampling configuration per batch
        if any(r[k] != first[k] for k in ("temperature", "top_p", "top_k", "max_tokens", "apply_chat_template", "add_generation_prompt", "enable_thinking")):
            print("error: streamed batches share their sampling settings; split the file", file=sys.stderr)
            return 2
    tok = rt.Tokenizer.load_from_hf(a.model_dir)
    llm = LLM(a.model_dir, device=a.device, max_batch_size=a.max_batch_size or min(len(reqs), 8), max_input_len=a.max_input_len,
              max_kv_cache_capacity=a.max_kv_cache_capacity, tokenizer=tok, enable_in_flight_batching=True)
    try:
        if llm.native_runtime is None:
            print("error: the native runtime needs the native tokenizer (tokenizer.json)", file=sys.stderr)
            return 2
        req = rt.LLMGenerationRequest()
        entries = []
        for r in reqs:
            e = rt.GenerationEntry()
            if r["apply_chat_template"]:
                from ..chat_template import ChatTemplate
                e.prompt_ids = list(tok.encode(ChatTemplate.load(a.model_dir).apply(r["messages"], r["add_generation_prompt"],
                                                                                    enable_thinking=r["enable_thinking"])))
            else:
                e.prompt = "\n".join(str(m["content"]) for m in r["messages"])
            entries.append(e)
        req.requests = entries
        req.max_generate_length, req.temperature, req.top_k, req.top_p = first["max_tokens"], first["temperature"], first["top_k"], first["top_p"]
        req.seed, req.stop = first["seed"], [s for r in reqs for s in r["stop"]]
        req.apply_chat_template = False    # rendered above with the full (Jinja) template engine

        def on_tokens(i, tokens, text, finished):
            if a.plain:
                sys.stdout.write(text)
            elif text or tokens:
                sys.stdout.write(json.dumps({"request": i, "text": text, "tokens": list(tokens)}, ensure_ascii=False) + "\n")
            sys.stdout.flush()

        resp = llm.native_runtime.handle_request(req, on_tokens)
        if a.plain:
            sys.stdout.write("\n")
        else:
            for i, (reason, st, err) in enumerate(zip(resp.finish_reasons, resp.stats, resp.errors)):
                sys.stdout.write(json.dumps({"request": i, "finished": True, "finish_reason": str(reason).split(".")[-1], "error": err,
                                             "prompt_tokens": st.prompt_tokens, "generated_tokens": st.generated_tokens,
                                             "ttft_ms": round(st.ttft_s * 1e3, 3), "total_ms": round(st.total_s * 1e3, 3)}) + "\n")
        return 0 if not any(resp.errors) else 1
    finally:
        llm.close()


if __name__ == "__main__":
    sys.exit(main())
