"""Offline benchmark with a machine-readable report (``python -m tensorrt_edge_llm_b200.benchmarks.llm_bench``).

Counterpart of the reference's ``examples/cpp/llm_bench.cpp``: modes ``generate`` (prefill + ``--osl`` decode tokens
per iteration) and ``fixed_round`` (``--osl`` decode rounds on a context of ``--input-len`` tokens, prefill untimed),
options ``--input-len --batch-size --osl --warmup --iterations --force-al --seed --no-gpu-timing`` (:141-154), and a
``report.json`` (schema version 2, :420-489) holding per-iteration samples, their statistics (population standard
deviation, upper median, ``sorted[min(floor(N·p), N-1)]`` percentiles), stage timings, peak device memory and FNV-1a
fingerprints of the generated tokens."""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time
from typing import Dict, List

import torch

from .. import profiling as prof
from .._version import __version__


def fnv1a64(data: bytes) -> str:
    h = 0xcbf29ce484222325
    for b in data:
        h = ((h ^ b) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return f"{h:016x}"


def summarize(values: List[float]) -> Dict[str, float]:
    if not values:
        return {}
    v = sorted(values)
    n = len(v)
    mean = sum(v) / n

    def pct(p):
        return v[min(int(math.floor(n * p)), n - 1)]
    return {"count": n, "mean": mean, "stddev": math.sqrt(sum((x - mean) ** 2 for x in v) / n), "min": v[0], "max": v[-1],
            "median": v[n // 2], "p90": pct(0.90), "p95": pct(0.95), "p99": pct(0.99)}


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="llm_bench")
    p.add_argument("--model", default="", help="checkpoint directory; empty = random weights of --shape")
    p.add_argument("--shape", default="tiny", choices=["tiny", "qwen3-8b"])
    p.add_argument("--layers", type=int, default=0)
    p.add_argument("--dtype", default="", choices=["", "float32", "bfloat16", "float16"])
    p.add_argument("--quantization", default="", choices=["", "nvfp4"])
    p.add_argument("--mode", default="generate", choices=["generate", "fixed_round"])
    p.add_argument("--input-len", "--inputLen", type=int, default=128)
    p.add_argument("--batch-size", "--batchSize", type=int, default=1)
    p.add_argument("--osl", type=int, default=32)
    p.add_argument("--warmup", type=int, default=1)
    p.add_argument("--iterations", type=int, default=3)
    p.add_argument("--force-al", "--forceAl", type=float, default=0.0, help="forced acceptance length (speculative runs)")
    p.add_argument("--seed", type=int, default=1234)
    p.add_argument("--no-gpu-timing", "--noGpuTiming", action="store_true")
    p.add_argument("--ignore-eos", "--ignoreEos", action="store_true", default=True)
    p.add_argument("--device", default="")
    p.add_argument("--output-dir", "--outputDir", default="llm_bench_out")
    return p


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    from ..config import qwen3_8b_config, tiny_llama_config
    from ..runtime.llm import LLM, SamplingParams
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    gpu_timing = dev.startswith("cuda") and not a.no_gpu_timing
    os.makedirs(a.output_dir, exist_ok=True)
    report = {"schema_version": 2, "runtime_version": __version__, "mode": a.mode, "status": "failed",
              "deployment": {"model": a.model or a.shape, "batch_size": a.batch_size, "input_len": a.input_len, "osl": a.osl,
                             "quantization": a.quantization or "none", "device": dev},
              "gpu": torch.cuda.get_device_name(0) if dev.startswith("cuda") else "cpu", "torch_version": torch.__version__,
              "cuda_runtime_version": torch.version.cuda, "warmup": a.warmup, "iterations": a.iterations, "ignore_eos": a.ignore_eos,
              "forced_acceptance_length": a.force_al, "gpu_timing": gpu_timing,
              "statistics_definition": "population stddev; upper median; sorted[min(floor(N*p),N-1)] percentile"}
    samples: List[dict] = []
    try:
        if a.model:
            model = a.model
        else:
            kw = {"num_hidden_layers": a.layers} if a.layers else {}
            if a.dtype:
                kw["dtype"] = a.dtype
            model = (tiny_llama_config if a.shape == "tiny" else qwen3_8b_config)(**kw)
            if a.quantization == "nvfp4":
                from ..config import QUANT_NVFP4, QuantConfig
                model.quant = QuantConfig(quant_type=QUANT_NVFP4, group_size=16)
        cap = a.input_len + a.osl + 64
        llm = LLM(model, device=dev, max_batch_size=a.batch_size, max_input_len=a.input_len, max_kv_cache_capacity=cap,
                  max_num_tokens=max(8192, a.input_len))
        report["engine_config"] = {k: v for k, v in vars(llm.cfg).items() if isinstance(v, (int, float, str, bool, type(None)))}
        g = torch.Generator().manual_seed(a.seed)
        prompts = torch.randint(3, llm.cfg.vocab_size, (a.batch_size, a.input_len), generator=g).tolist()
        sp = SamplingParams(max_tokens=a.osl, temperature=0.0, ignore_eos=a.ignore_eos)
        report["workloads"] = [{"batch_size": a.batch_size, "input_len": a.input_len, "osl": a.osl, "seed": a.seed}]
        prof.set_profiling_enabled(True)
        monitor = prof.MemoryMonitor().start()
        token_bytes = b""
        for it in range(a.warmup + a.iterations):
            prof.timer().reset()
            if gpu_timing:
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            t0 = time.perf_counter()
            outs = llm.generate(prompts, sp)
            if gpu_timing:
                e1.record()
                torch.cuda.synchronize()
                total_ms = e0.elapsed_time(e1)
            else:
                total_ms = (time.perf_counter() - t0) * 1e3
            if it < a.warmup:
                continue
            stages = prof.timer().summary()
            prefill_ms = stages.get(prof.PREFILL, {}).get("total_ms", outs[0].ttft_s * 1e3)
            decode_ms = stages.get(prof.VANILLA_DECODING, {}).get("total_ms", outs[0].decode_s * 1e3)
            n_out = sum(len(o.token_ids) for o in outs)
            timed_ms = decode_ms if a.mode == "fixed_round" else total_ms
            samples.append({"iteration": it - a.warmup, "total_ms": total_ms, "prefill_ms": prefill_ms, "decode_ms": decode_ms,
                            "output_tokens": n_out, "output_tokens_per_s": n_out / (timed_ms / 1e3) if timed_ms > 0 else 0.0,
                            "ms_per_decode_round": decode_ms / max(a.osl - 1, 1),
                            "stages": {k: round(v["total_ms"], 4) for k, v in stages.items()}})
            token_bytes = b"".join(torch.tensor(o.token_ids, dtype=torch.int32).numpy().tobytes() for o in outs)
        report["peak_device_memory_bytes"] = monitor.stop()
        report["memory_source"] = monitor.source
        report["samples"] = samples
        report["statistics"] = {k: summarize([s[k] for s in samples]) for k in ("total_ms", "prefill_ms", "decode_ms", "output_tokens_per_s",
                                                                                "ms_per_decode_round")}
        report["fingerprints"] = {"algorithm": "FNV-1a-64, noncryptographic", "representation": "16 lowercase hexadecimal digits",
                                  "token_encoding": "per-sequence int32 token IDs, little-endian bytes, no separators",
                                  "output_tokens": fnv1a64(token_bytes)}
        report["status"] = "complete"
        llm.close()
    except Exception as e:       # the report still records what ran before the failure
        report["error"] = f"{type(e).__name__}: {e}"
        report["samples"] = samples
    finally:
        prof.set_profiling_enabled(False)
    with open(os.path.join(a.output_dir, "report.json"), "w", encoding="utf-8") as f:
        json.dump(report, f, indent=2)
    print(json.dumps(report.get("statistics", {"error": report.get("error")}), indent=2))
    print("Benchmark report:", os.path.join(a.output_dir, "report.json"))
    return 0 if report["status"] == "complete" else 1


if __name__ == "__main__":
    sys.exit(main())
