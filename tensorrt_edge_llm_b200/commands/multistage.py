"""``trtedge multistage``: run requests through the stage graph of an engine directory
(the reference's ``examples/cpp/multistage_inference.cpp``: ``--config --prompt --input-file --output-file
--batch-size --validate-config``)."""
from __future__ import annotations

import argparse
import json


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge multistage")
    p.add_argument("--config", required=True, help="directory holding multistage_config.json (or the file itself)")
    p.add_argument("--prompt", default=None)
    p.add_argument("--input-file", "--inputFile", default=None, help="JSON: {\"requests\": [{\"messages\": [...]}, ...]}")
    p.add_argument("--output-file", "--outputFile", default=None)
    p.add_argument("--batch-size", "--batchSize", type=int, default=1)
    p.add_argument("--sampling", default=None, help="JSON object of default sampling settings")
    p.add_argument("--validate-config", "--validateConfig", action="store_true")
    p.add_argument("--write-one-stage-graph", action="store_true", help="write the one-stage graph of a plain LLM directory and exit")
    a = p.parse_args(argv)
    from ..runtime import multistage as ms
    if a.write_one_stage_graph:
        print(ms.write_graph(a.config, ms.one_stage_graph()))
        return 0
    try:
        graph = ms.load_graph(a.config)
    except (ms.GraphConfigError, OSError, json.JSONDecodeError) as e:
        print(f"invalid graph: {e}")
        return 1
    if a.validate_config:
        print("graph ok; execution order:", " -> ".join(ms.validate_graph(graph)))
        return 0
    default_sampling = json.loads(a.sampling) if a.sampling else None
    if a.input_file:
        with open(a.input_file, "r", encoding="utf-8") as f:
            body = json.load(f)
        requests = body["requests"] if isinstance(body, dict) else body
    elif a.prompt is not None:
        requests = [{"messages": [{"role": "user", "content": a.prompt}]}]
    else:
        p.error("give --prompt, --input-file or --validate-config")
    for r in requests:
        if default_sampling and "sampling" not in r:
            r["sampling"] = default_sampling
    rt = ms.MultiStageRuntime(graph)
    try:
        results = rt.run(requests, batch_size=a.batch_size)
    finally:
        rt.close()
    if a.output_file:
        with open(a.output_file, "w", encoding="utf-8") as f:
            json.dump({"responses": results}, f, indent=1)
    for i, r in enumerate(results):
        print(f"[{i}] ok={r['ok']}", r["outputs"] if r["ok"] else r["error"])
    return 0 if all(r["ok"] for r in results) else 1
