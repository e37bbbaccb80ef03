#!/usr/bin/env python
"""Headline benchmark: output tokens/s (whole job) + p50 TTFT / TPOT of a Qwen3-8B-shape decoder,
NVFP4 weights (or bf16), batch B, 1024 input / 128 output tokens, greedy, 64-token KV pages,
tensor parallel over N GPUs of one node.

One *step* is one complete request batch: prefill of B x 1024 tokens followed by 127 decode
steps (the first output token comes from the prefill), i.e. B x 128 output tokens.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...        # the unmodified reference, if it can run here

Rank 0 prints ONE JSON line.  `value` is device-timed (CUDA events, max over ranks) with inputs
resident on the device; `e2e` repeats the measurement through the public `LLM.generate` call with
prompts in pinned host memory (H2D every step) and the generated tokens read back (D2H).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_NOTE = "published reference numbers exist only for Jetson/GB10 (none for B200); vs_baseline is null"


def _reference_arm(args) -> int:
    """The reference needs TensorRT 11 engines + its plugin library; neither TensorRT nor a way to
    build its wheel (CMake < 4, scikit-build-core < 0.12, nanobind-backend) exists in this image."""
    reason = ("reference cannot be installed offline: pip metadata step fails (scikit-build-core needs CMake <4, "
              "image has 4.4.3; nanobind-backend and TensorRT 11 absent), and its runtime executes TensorRT engines")
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "tensorrt_edgellm")
    if os.path.isdir(ref_dir):
        try:
            import tensorrt  # noqa: F401
        except Exception:
            reason = "reference package present but TensorRT is not installed: its runtime only executes TensorRT engines"
    print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap", nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                 nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake"}
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense", choices=["dense", "moe", "hybrid", "eagle", "serve"],
                    help="dense = the headline benchmark; moe / hybrid / eagle are the secondary configurations; serve = the request engine "
                         "with staggered arrivals (in-flight batching)")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--input-len", type=int, default=None)
    ap.add_argument("--output-len", type=int, default=None)
    ap.add_argument("--dtype", default="nvfp4", choices=["nvfp4", "bf16", "fp16"])
    ap.add_argument("--layers", type=int, default=None, help="debug only; anything but the full depth is not the named config")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--kv-cache-dtype", default="model", choices=["model", "fp8"],
                    help="KV page storage; anything but the default (the compute type) is not the named headline configuration")
    args = ap.parse_args()
    if args.impl == "reference":
        return _reference_arm(args)
    if args.workload != "dense":
        from tensorrt_edge_llm_b200.benchmarks.workloads import main as workload_main
        return workload_main(args)
    args.batch, args.input_len, args.output_len = args.batch or 64, args.input_len or 1024, args.output_len or 128
    args.layers = args.layers or 36

    import torch
    import torch.distributed as dist
    from tensorrt_edge_llm_b200.config import QUANT_NVFP4, QuantConfig, qwen3_8b_config
    from tensorrt_edge_llm_b200.ops import cuda as cu
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE {world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from tensorrt_edge_llm_b200.parallel import make_comm
        comm = make_comm(args.comm, dev)

    act = "float16" if args.dtype in ("nvfp4", "fp16") else "bfloat16"
    quant = QuantConfig(quant_type=QUANT_NVFP4, group_size=16) if args.dtype == "nvfp4" else QuantConfig()
    cfg = qwen3_8b_config(dtype=act, quant=quant, num_hidden_layers=args.layers)
    if world > 1:
        cfg = cfg.for_rank(rank, world)
    B, S, O = args.batch, args.input_len, args.output_len
    llm = LLM(cfg, device=str(dev), comm=comm, max_batch_size=B, max_input_len=S, max_kv_cache_capacity=S + O + 64,
              page_size=64, max_num_tokens=8192, random_init_seed=0, kv_cache_dtype=args.kv_cache_dtype)
    runner, kv = llm.runner, llm.kv
    g = torch.Generator().manual_seed(1234)
    prompts_host = torch.randint(0, cfg.vocab_size, (B, S), generator=g, dtype=torch.int32).pin_memory()
    prompts_dev = prompts_host.to(dev)
    seats = list(range(B))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # > 126 MB L2

    def one_batch_device():
        """prefill + decode with device-resident inputs; returns (prefill_ms, decode_ms)."""
        for s in seats:
            kv.free(s)
            kv.reserve(s, S + O)
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        logits = runner.prefill_tensor(seats, prompts_dev)
        first = runner.sample(logits, SamplingParams(), 0)
        e1.record()
        toks = runner.decode_greedy(seats, first, O - 1)
        e2.record()
        return e0, e1, e2, toks

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        one_batch_device()
        flush.fill_(1)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = cu.LAUNCHES
    step_ms, pre_ms, dec_ms = [], [], []
    for _ in range(args.steps):
        flush.fill_(0)
        barrier()
        e0, e1, e2, toks = one_batch_device()
        barrier()
        step_ms.append(e0.elapsed_time(e2))
        pre_ms.append(e0.elapsed_time(e1))
        dec_ms.append(e1.elapsed_time(e2))
    launches = cu.LAUNCHES - launches0
    clocks = sampler.stop()
    cu.Workspace.get(dev).check_status()

    # ---- N > 1: the same timed loop with every collective through NCCL (all-reduce, then the local norm kernel; a small
    # all-gather of per-shard candidates for the greedy pick).  The reference cannot run on this image, so this is the
    # composition its AllReducePlugin → ncclAllReduce path amounts to, on the same model, kernels and box.
    nccl_arm = None
    if world > 1 and args.comm == "fused" and hasattr(comm, "force_nccl"):
        comm.force_nccl = True
        runner._graphs.clear()
        for _ in range(max(2, min(args.warmup, 3))):
            one_batch_device()
            flush.fill_(1)
        n_ms, n_pre, n_dec = [], [], []
        for _ in range(args.steps):
            flush.fill_(0)
            barrier()
            e0, e1, e2, _t = one_batch_device()
            barrier()
            n_ms.append(e0.elapsed_time(e2))
            n_pre.append(e0.elapsed_time(e1))
            n_dec.append(e1.elapsed_time(e2))
        nccl_arm = (sum(n_ms) / len(n_ms), statistics.median(n_pre), statistics.median(n_dec))
        comm.force_nccl = False
        runner._graphs.clear()
        cu.Workspace.get(dev).check_status()

    # ---- end to end through the public API: pinned host prompts in, generated tokens out --------
    sp = SamplingParams(max_tokens=O, ignore_eos=True)
    e2e_s, ttft, tpot = [], [], []
    llm.generate(prompts_host, sp)
    for _ in range(max(1, args.steps)):
        flush.fill_(0)
        barrier()
        t0 = time.perf_counter()
        outs = llm.generate(prompts_host, sp)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        e2e_s.append(t1 - t0)
        ttft.append(outs[0].ttft_s)
        tpot.append(outs[0].decode_s / max(1, O - 1))
    assert all(len(o.token_ids) == O for o in outs)

    def maxr(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms = maxr(sum(step_ms) / len(step_ms))
    e2e = maxr(sum(e2e_s) / len(e2e_s))
    value = B * O / (ms / 1e3)
    out = {
        "metric": "output tok/s (whole box), Qwen3-8B-shape, 1024 in / 128 out; p50 TTFT/TPOT in config",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "nvfp4-weights/nvfp4-act-gemm/fp16-activations" if args.dtype == "nvfp4" else args.dtype,
        "data": "synthetic (seeded uniform token ids, random-init N(0,0.02) weights)",
        "config": {"model": "Qwen3-8B-shape (36L, H4096, 32q/8kv, d128, I12288, V151936)" if args.layers == 36 else f"DEBUG {args.layers} layers",
                   "global_batch": B, "seq_len": S, "output_len": O, "parallelism": f"tp{world}", "page_size": 64,
                   "weights": args.dtype, "kv_cache": args.kv_cache_dtype, "comm": args.comm if world > 1 else "none",
                   "l2": "256 MiB buffer written between timed steps; weights (>= 4.6 GB) exceed L2 every decode step",
                   "prefill_ms": round(maxr(statistics.median(pre_ms)), 3),
                   "decode_ms_per_token": round(maxr(statistics.median(dec_ms)) / max(1, O - 1), 4),
                   "p50_ttft_ms": round(maxr(statistics.median(ttft)) * 1e3, 3),
                   "p50_tpot_ms": round(maxr(statistics.median(tpot)) * 1e3, 4),
                   "baseline_note": BASELINE_NOTE},
        "clocks": clocks,
        "e2e": {"value": round(B * O / e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": int(prompts_host.numel() * 4),
                "d2h_bytes_per_step": int(B * O * 4), "ms_per_step": round(e2e * 1e3, 3)},
        "gpu_launches": int(launches),
    }
    if nccl_arm is not None:
        n_ms = maxr(nccl_arm[0])
        out["nccl_arm"] = {"value": round(B * O / (n_ms / 1e3), 1), "unit": "tok/s", "ms_per_step": round(n_ms, 3),
                           "prefill_ms": round(maxr(nccl_arm[1]), 3), "decode_ms_per_token": round(maxr(nccl_arm[2]) / max(1, O - 1), 4),
                           "what": "same model and kernels, every collective through NCCL (torch.distributed) instead of the fused peer-memory kernels"}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        # Captured graphs hold NCCL kernels; tearing the communicator down under them can block, so
        # the ranks synchronise once more and leave without the collective destructor.
        llm.runner._graphs.clear()
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
