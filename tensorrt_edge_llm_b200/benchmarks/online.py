"""Online (HTTP) benchmark: replay a workload against a running server and report latency percentiles.

A workload is a JSON file ``{"requests": [{"at_s": 0.0, "prompt": "...", "max_tokens": 64, "priority": 0}, ...]}`` (or a
generated one: ``--num-requests N --rate R --prompt-len P --max-tokens T``).  Requests are fired at their arrival
times over the streaming chat-completions route; per request the client records time to first token, inter-token
gaps and end-to-end latency.  The report carries p50 / p95 / p99 of each, request throughput and
``output_tokens_per_s`` over the whole run.

Parity: ``scripts/benchmark_runner`` (``metrics.py:21-74``, ``__main__.py:27-35``) of the reference."""
from __future__ import annotations

import argparse
import asyncio
import json
import random
import statistics
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class RequestRecord:
    at_s: float
    ttft_s: Optional[float] = None
    latency_s: Optional[float] = None
    gaps_s: List[float] = field(default_factory=list)
    output_tokens: int = 0
    status: int = 0
    error: str = ""


def percentile(values: List[float], q: float) -> Optional[float]:
    """Linear-interpolated percentile (q in [0, 100]); None for an empty list."""
    if not values:
        return None
    v = sorted(values)
    pos = (len(v) - 1) * q / 100.0
    lo, hi = int(pos), min(int(pos) + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (pos - lo)


def summarize(records: List[RequestRecord], wall_s: float) -> Dict:
    ok = [r for r in records if r.error == "" and r.latency_s is not None]
    gaps = [g for r in ok for g in r.gaps_s]

    def stats(vals):
        return {"p50": percentile(vals, 50), "p95": percentile(vals, 95), "p99": percentile(vals, 99),
                "mean": statistics.fmean(vals) if vals else None}

    by_status: Dict[str, int] = {}
    for r in records:
        by_status[str(r.status)] = by_status.get(str(r.status), 0) + 1
    return {"requests": len(records), "completed": len(ok), "failed": len(records) - len(ok), "status_counts": by_status,
            "wall_s": wall_s, "requests_per_s": len(ok) / wall_s if wall_s > 0 else None,
            "output_tokens": sum(r.output_tokens for r in ok),
            "output_tokens_per_s": sum(r.output_tokens for r in ok) / wall_s if wall_s > 0 else None,
            "ttft_s": stats([r.ttft_s for r in ok if r.ttft_s is not None]), "latency_s": stats([r.latency_s for r in ok]),
            "inter_token_s": stats(gaps)}


def synthetic_workload(num_requests: int, rate: float, prompt_len: int, max_tokens: int, seed: int = 0) -> List[dict]:
    """Poisson arrivals at ``rate`` requests / s (all at t = 0 when rate <= 0) with prompts of ``prompt_len`` words."""
    rng = random.Random(seed)
    t, out = 0.0, []
    for i in range(num_requests):
        if rate > 0 and i:
            t += rng.expovariate(rate)
        words = " ".join(rng.choice(("alpha", "beta", "gamma", "delta", "tensor", "kernel", "token")) for _ in range(prompt_len))
        out.append({"at_s": t, "prompt": words, "max_tokens": max_tokens})
    return out


async def _one(client, url: str, model: str, req: dict, t0: float, headers: dict) -> RequestRecord:
    rec = RequestRecord(at_s=req.get("at_s", 0.0))
    delay = rec.at_s - (time.perf_counter() - t0)
    if delay > 0:
        await asyncio.sleep(delay)
    body = {"model": model, "messages": [{"role": "user", "content": req["prompt"]}], "max_tokens": req.get("max_tokens", 64),
            "temperature": req.get("temperature", 0.0), "stream": True, "priority": req.get("priority", 0)}
    start = last = time.perf_counter()
    try:
        async with client.stream("POST", url, json=body, headers=headers) as resp:
            rec.status = resp.status_code
            if resp.status_code != 200:
                rec.error = (await resp.aread()).decode("utf-8", "replace")[:200]
                return rec
            async for line in resp.aiter_lines():
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                chunk = json.loads(line[6:])
                if "error" in chunk:
                    rec.error = str(chunk["error"])[:200]
                    break
                now = time.perf_counter()
                choice = chunk["choices"][0]
                if choice["delta"].get("content"):
                    if rec.ttft_s is None:
                        rec.ttft_s = now - start
                    else:
                        rec.gaps_s.append(now - last)
                    last = now
                if chunk.get("usage"):
                    rec.output_tokens = chunk["usage"]["completion_tokens"]
        rec.latency_s = time.perf_counter() - start
    except Exception as e:          # connection errors are data points, not crashes
        rec.error = f"{type(e).__name__}: {e}"[:200]
    return rec


async def run_workload(requests: List[dict], base_url: str = "http://127.0.0.1:8000", model: str = "model", api_key: str = "",
                       client=None) -> Dict:
    import httpx
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    own = client is None
    client = client or httpx.AsyncClient(timeout=None)
    t0 = time.perf_counter()
    try:
        recs = await asyncio.gather(*[_one(client, base_url.rstrip("/") + "/v1/chat/completions", model, r, t0, headers) for r in requests])
    finally:
        if own:
            await client.aclose()
    return summarize(list(recs), time.perf_counter() - t0)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m tensorrt_edge_llm_b200.benchmarks.online")
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="model")
    ap.add_argument("--api-key", default="")
    ap.add_argument("--workload", default="", help="JSON workload file; otherwise a synthetic one is generated")
    ap.add_argument("--num-requests", type=int, default=32)
    ap.add_argument("--rate", type=float, default=0.0, help="mean arrivals per second (0 = all at once)")
    ap.add_argument("--prompt-len", type=int, default=64)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--output", default="")
    a = ap.parse_args(argv)
    if a.workload:
        with open(a.workload, "r", encoding="utf-8") as f:
            reqs = json.load(f)["requests"]
    else:
        reqs = synthetic_workload(a.num_requests, a.rate, a.prompt_len, a.max_tokens)
    report = asyncio.run(run_workload(reqs, a.base_url, a.model, a.api_key))
    text = json.dumps(report, indent=1)
    if a.output:
        with open(a.output, "w", encoding="utf-8") as f:
            f.write(text)
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
