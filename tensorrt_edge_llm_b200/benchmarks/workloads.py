"""Secondary benchmark workloads (one GPU, or one process per GPU under torchrun for moe / hybrid / eagle): the MoE, hybrid and speculative-decoding configurations that sit
next to the dense headline benchmark.  Each prints one JSON line with device-timed numbers (CUDA events after
warm-up, synthetic seeded token ids, random-init weights of the named architecture).

    python bench.py --workload moe      # Qwen3-30B-A3B shape, NVFP4 experts, batch 32, 2048 in / 256 out
    python bench.py --workload hybrid   # Nemotron-H-style Mamba2 + gated DeltaNet + attention, batch 16, 8192 in / 256 out
    python bench.py --workload eagle    # EAGLE-3 tree speculative decoding on the Qwen3-8B shape, forced accept lengths
    python bench.py --workload serve    # the served path: native request engine, staggered arrivals, in-flight batching
"""
from __future__ import annotations

import json
import statistics
import time

import torch


def _events(n):
    return [torch.cuda.Event(enable_timing=True) for _ in range(n)]


def _generate_timed(llm, prompts_dev, out_len, steps, warmup):
    from ..runtime.runner import SamplingParams
    runner, kv = llm.runner, llm.kv
    b, s = prompts_dev.shape
    seats = list(range(b))
    pre, dec = [], []
    for it in range(warmup + steps):
        for seat in seats:
            kv.free(seat)
            kv.reserve(seat, s + out_len)
        e0, e1, e2 = _events(3)
        e0.record()
        logits = runner.prefill_tensor(seats, prompts_dev)
        first = runner.sample(logits, SamplingParams(), 0)
        e1.record()
        runner.decode_greedy(seats, first, out_len - 1)
        e2.record()
        torch.cuda.synchronize()
        if it >= warmup:
            pre.append(e0.elapsed_time(e1))
            dec.append(e1.elapsed_time(e2))
    return statistics.median(pre), statistics.median(dec)


def _dist():
    """(rank, world, device, comm) — one process per GPU under torchrun, else a single GPU."""
    import os
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from ..parallel import make_comm
        comm = make_comm("fused", dev)
    return rank, world, dev, comm


def run_moe(args) -> dict:
    from ..config import QUANT_NVFP4, QuantConfig, qwen3_30b_a3b_config
    from ..ops import cuda as cu
    from ..runtime.llm import LLM
    b, s, o = args.batch or 32, args.input_len or 2048, args.output_len or 256
    rank, world, dev, comm = _dist()
    quant = QuantConfig(quant_type=QUANT_NVFP4, group_size=16, excluded=["*self_attn*", "*mlp.gate", "lm_head"])
    cfg = qwen3_30b_a3b_config(dtype="bfloat16", quant=quant, **({"num_hidden_layers": args.layers} if args.layers else {}))
    if world > 1:
        cfg = cfg.for_rank(rank, world, ep=True)       # attention tensor-parallel, experts sharded by id
    llm = LLM(cfg, device=str(dev), comm=comm, max_batch_size=b, max_input_len=s, max_kv_cache_capacity=s + o + 64, max_num_tokens=8192)
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (b, s), generator=g, dtype=torch.int32).to(dev)
    l0 = cu.LAUNCHES
    pre, dec = _generate_timed(llm, prompts, o, args.steps, args.warmup)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([pre, dec], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pre, dec = float(t[0]), float(t[1])
    ms = pre + dec
    return {"metric": "output tok/s, Qwen3-30B-A3B-shape MoE (48L, H2048, 128 experts top-8, I768), NVFP4 experts + bf16 attention",
            "value": round(b * o / (ms / 1e3), 1), "unit": "tok/s", "n_gpus": world, "ms_per_step": round(ms, 3),
            "config": {"global_batch": b, "seq_len": s, "output_len": o, "prefill_ms": round(pre, 3),
                       "decode_ms_per_token": round(dec / max(1, o - 1), 4), "parallelism": f"tp{world}-attention + ep{world}-experts",
                       "layers": cfg.num_hidden_layers, "ep_all_to_all": bool(comm is not None and getattr(comm, "_ep", None))},
            "gpu_launches": int(cu.LAUNCHES - l0), "data": "synthetic", "_rank": rank, "_world": world, "_llm": llm}


def _max_over_ranks(world, dev, *vals):
    if world <= 1:
        return vals
    import torch.distributed as dist
    t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return tuple(float(v) for v in t)


def run_hybrid(args) -> dict:
    from ..config import hybrid_nemotron_config
    from ..ops import cuda as cu
    from ..runtime.llm import LLM
    b, s, o = args.batch or 16, args.input_len or 8192, args.output_len or 256
    rank, world, dev, comm = _dist()
    cfg = hybrid_nemotron_config(dtype="bfloat16", **({"num_hidden_layers": args.layers} if args.layers else {}))
    if world > 1:
        cfg = cfg.for_rank(rank, world)
    # recurrent layers walk a sequence in order, so prefill chunks carry several sequences side by side
    llm = LLM(cfg, device=str(dev), comm=comm, max_batch_size=b, max_input_len=s, max_kv_cache_capacity=s + o + 64, max_num_tokens=4 * 8192)
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (b, s), generator=g, dtype=torch.int32).to(dev)
    l0 = cu.LAUNCHES
    pre, dec = _generate_timed(llm, prompts, o, args.steps, args.warmup)
    pre, dec = _max_over_ranks(world, dev, pre, dec)
    ms = pre + dec
    return {"metric": "output tok/s, Nemotron-H-style hybrid (Mamba2 + gated DeltaNet + GQA attention), bf16",
            "value": round(b * o / (ms / 1e3), 1), "unit": "tok/s", "n_gpus": world, "ms_per_step": round(ms, 3),
            "config": {"global_batch": b, "seq_len": s, "output_len": o, "prefill_ms": round(pre, 3),
                       "decode_ms_per_token": round(dec / max(1, o - 1), 4), "layers": cfg.num_hidden_layers, "parallelism": f"tp{world}",
                       "layer_types": {t: cfg.layer_types.count(t) for t in sorted(set(cfg.layer_types))}},
            "gpu_launches": int(cu.LAUNCHES - l0), "data": "synthetic", "_rank": rank, "_world": world, "_llm": llm}


def run_eagle(args) -> dict:
    from ..config import qwen3_8b_config
    from ..model import AutoModel
    from ..ops import cuda as cu
    from ..runtime.kv_cache import KVCacheManager
    from ..runtime.runner import ModelRunner
    from ..runtime.speculative import EagleDecoder, SpecConfig
    b, s, rounds = args.batch or 4, args.input_len or 2048, args.output_len or 32
    rank, world, dev, comm = _dist()
    kw = {"num_hidden_layers": args.layers} if args.layers else {}
    cfg = qwen3_8b_config(dtype="bfloat16", **kw)
    if world > 1:                   # the target is tensor-parallel; the one-layer draft runs replicated on every rank
        cfg = cfg.for_rank(rank, world)
    model = AutoModel.from_config(cfg, device=dev, random_init=0, **({"comm": comm} if comm is not None else {}))
    dcfg = qwen3_8b_config(dtype="bfloat16", num_hidden_layers=1)
    dcfg.draft_type, dcfg.eagle3_target_hidden_size, dcfg.has_qk_norm = "eagle3", cfg.hidden_size, False
    draft = AutoModel.from_config(dcfg, device=dev, random_init=1)
    pages = (s + rounds * 8 + 256) // 64 + 2
    kv = KVCacheManager(cfg, num_pages=pages * b + 1, page_size=64, max_seats=b, max_pages_per_seq=pages, device=dev)
    dkv = KVCacheManager(dcfg, num_pages=pages * b + 1, page_size=64, max_seats=b, max_pages_per_seq=pages, device=dev, num_layers=1)
    runner = ModelRunner(model, kv, max_num_tokens=8192)
    runner.use_cuda_graphs = False
    spec = SpecConfig(draft_steps=6, top_k=10, verify_tokens=60, force_accept_mean=3.5, force_seed=0)
    dec = EagleDecoder(runner, draft, dkv, spec)
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (b, s), generator=g).tolist()
    seats = list(range(b))
    l0 = cu.LAUNCHES
    t0 = time.perf_counter()
    dec.prefill(seats, prompts)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for _ in range(args.warmup):
        dec.round(seats)
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    emitted0, r0 = dec.stats.emitted, dec.stats.rounds
    e0, e1 = _events(2)
    e0.record()
    for _ in range(rounds):
        dec.round(seats)
    e1.record()
    torch.cuda.synchronize()
    (ms,) = _max_over_ranks(world, dev, e0.elapsed_time(e1))
    emitted = dec.stats.emitted - emitted0
    return {"metric": "output tok/s, EAGLE-3 tree speculative decoding on the Qwen3-8B shape (bf16), top-k 10, depth 6, 60 verify tokens",
            "value": round(emitted / (ms / 1e3), 1), "unit": "tok/s", "n_gpus": world, "ms_per_round": round(ms / rounds, 3),
            "config": {"global_batch": b, "prompt_len": s, "rounds": rounds, "mean_accept_length": round(emitted / (rounds * b), 3),
                       "forced_accept_mean": 3.5, "prefill_s": round(t1 - t0, 3), "draft_forwards_per_round": spec.draft_steps,
                       "layers": cfg.num_hidden_layers, "parallelism": f"tp{world} target, replicated draft",
                       "note": "eager rounds; tree mask, positions and verify-tree selection are built on the device, one "
                               "device→host read per round (accepted path); accept lengths are prescribed"},
            "gpu_launches": int(cu.LAUNCHES - l0), "data": "synthetic", "_rank": rank, "_world": world}


def run_serve(args) -> dict:
    """The served path: requests arrive one by one at the native request engine (``csrc/runtime/scheduler.cpp``), are
    admitted mid-flight into at most ``batch`` seats, prefilled in chunks next to the running decode rows and decoded by
    graph replays once a step holds decode rows only.  Reports whole-run output tokens/s (wall clock from the first
    submission to the last completion: arrivals are host events) and per-request p50 / p95 TTFT and TPOT from the
    engine's own request statistics.  Prompts are host-side token lists (copied to the device by every step that
    consumes them); every generated token is read back to the host by the step that produced it."""
    from ..config import QUANT_NVFP4, QuantConfig, qwen3_8b_config
    from ..ops import cuda as cu
    from ..runtime.llm import LLM
    from ..runtime.runner import SamplingParams
    b, s, o = args.batch or 64, args.input_len or 1024, args.output_len or 128
    n_req = max(1, args.steps) * b                    # `steps` waves of `batch` requests
    gap_s = 0.005                                     # one arrival every 5 ms (200 requests / s offered)
    act = "float16" if args.dtype in ("nvfp4", "fp16") else "bfloat16"
    quant = QuantConfig(quant_type=QUANT_NVFP4, group_size=16) if args.dtype == "nvfp4" else QuantConfig()
    cfg = qwen3_8b_config(dtype=act, quant=quant, **({"num_hidden_layers": args.layers} if args.layers else {}))
    llm = LLM(cfg, device="cuda", max_batch_size=b, max_input_len=s, max_kv_cache_capacity=s + o + 64, page_size=64,
              max_num_tokens=8192, random_init_seed=0, enable_in_flight_batching=True,
              scheduling={"mode": "mixed", "max_num_tokens": 8192, "max_chunk_tokens": 2048})
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (n_req, s), generator=g, dtype=torch.int32).tolist()
    sp = SamplingParams(max_tokens=o, ignore_eos=True)

    def wave(reqs, gap):
        t0 = time.perf_counter()
        handles = []
        for i, p in enumerate(reqs):
            while time.perf_counter() - t0 < i * gap:
                time.sleep(0.0005)
            handles.append(llm.submit(p, sp))
        outs = [h.get(600.0) for h in handles]
        torch.cuda.synchronize()
        return time.perf_counter() - t0, handles, outs
    # warm-up: a full wave (kernels, allocator) and every decode-graph bucket this seat count can reach
    for _ in range(max(1, min(args.warmup, 2))):
        wave(prompts[:b], 0.0)
    runner = llm.runner
    warm_seats = list(range(b))
    for seat in warm_seats:
        llm.kv.free(seat)
        llm.kv.reserve(seat, 8)
    for n in sorted({runner.graph_bucket(k) for k in range(1, b + 1)}):
        runner.decode_step_graph(warm_seats[:n], [1] * n)
    for seat in warm_seats:
        llm.kv.free(seat)
    torch.cuda.synchronize()
    l0, g0, m0 = cu.LAUNCHES, llm.session.graph_steps, llm.engine.metrics()
    wall, handles, outs = wave(prompts, gap_s)
    m1 = llm.engine.metrics()
    stats = [h.stats() for h in handles]
    ttft = sorted(st.ttft_s for st in stats)
    tpot = sorted((st.total_s - st.ttft_s) / max(1, st.generated_tokens - 1) for st in stats)
    pct = lambda xs, q: xs[min(len(xs) - 1, int(q * len(xs)))]
    total = sum(len(x) for x in outs)
    assert total == n_req * o
    cu.Workspace.get(torch.device("cuda", torch.cuda.current_device())).check_status()
    steps_all = (m1.decode_steps - m0.decode_steps) + (m1.prompt_steps - m0.prompt_steps) + (m1.mixed_steps - m0.mixed_steps)
    out = {"metric": "output tok/s through the request engine (in-flight batching, staggered arrivals), Qwen3-8B shape, 1024 in / 128 out",
           "value": round(total / wall, 1), "unit": "tok/s", "n_gpus": 1, "ms_per_step": round(wall * 1e3 / max(1, steps_all), 3),
           "config": {"requests": n_req, "seats": b, "seq_len": s, "output_len": o, "arrival_gap_ms": gap_s * 1e3, "weights": args.dtype,
                      "p50_ttft_ms": round(pct(ttft, 0.5) * 1e3, 2), "p95_ttft_ms": round(pct(ttft, 0.95) * 1e3, 2),
                      "p50_tpot_ms": round(pct(tpot, 0.5) * 1e3, 3), "p95_tpot_ms": round(pct(tpot, 0.95) * 1e3, 3),
                      "engine_steps": int(steps_all), "decode_only_steps": int(m1.decode_steps - m0.decode_steps),
                      "graph_replay_steps": int(llm.session.graph_steps - g0), "mixed_steps": int(m1.mixed_steps - m0.mixed_steps),
                      "admitted_mid_flight": int(m1.admitted_mid_flight - m0.admitted_mid_flight), "wall_s": round(wall, 3),
                      "layers": cfg.num_hidden_layers, "timing": "wall clock (arrivals are host events); per-request figures from the engine"},
           "e2e": {"value": round(total / wall, 1), "unit": "tok/s", "h2d_bytes_per_step": int(n_req * s * 4 / max(1, steps_all)),
                   "d2h_bytes_per_step": int(total * 4 / max(1, steps_all))},
           "gpu_launches": int(cu.LAUNCHES - l0), "data": "synthetic (seeded uniform token ids, random-init weights)",
           "dtype": "nvfp4-weights/nvfp4-act-gemm/fp16-activations" if args.dtype == "nvfp4" else args.dtype}
    llm.close()
    return out


def main(args) -> int:
    fn = {"moe": run_moe, "hybrid": run_hybrid, "eagle": run_eagle, "serve": run_serve}[args.workload]
    out = fn(args)
    rank, world, llm = out.pop("_rank", 0), out.pop("_world", 1), out.pop("_llm", None)
    out.update({"steps": args.steps, "warmup": args.warmup, "higher_is_better": True})
    out.setdefault("dtype", "bf16" if args.workload != "moe" else "nvfp4-experts/bf16")
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:       # graphs hold collective kernels: leave without the communicator's destructor
        import os
        import sys
        import torch.distributed as dist
        if llm is not None:
            llm.runner._graphs.clear()
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)
    return 0
