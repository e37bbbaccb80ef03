"""Secondary benchmark workloads (one GPU): the MoE, hybrid and speculative-decoding configurations that sit
next to the dense headline benchmark.  Each prints one JSON line with device-timed numbers (CUDA events after
warm-up, synthetic seeded token ids, random-init weights of the named architecture).

    python bench.py --workload moe      # Qwen3-30B-A3B shape, NVFP4 experts, batch 32, 2048 in / 256 out
    python bench.py --workload hybrid   # Nemotron-H-style Mamba2 + gated DeltaNet + attention, batch 16, 8192 in / 256 out
    python bench.py --workload eagle    # EAGLE-3 tree speculative decoding on the Qwen3-8B shape, forced accept lengths
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


def run_hybrid(args) -> dict:
    from ..config import hybrid_nemotron_config
    from ..ops import cuda as cu
    from ..runtime.llm import LLM
    b, s, o = args.batch or 16, args.input_len or 8192, args.output_len or 256
    cfg = hybrid_nemotron_config(dtype="bfloat16", **({"num_hidden_layers": args.layers} if args.layers else {}))
    # recurrent layers walk a sequence in order, so prefill chunks carry several sequences side by side
    llm = LLM(cfg, device="cuda", max_batch_size=b, max_input_len=s, max_kv_cache_capacity=s + o + 64, max_num_tokens=4 * 8192)
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (b, s), generator=g, dtype=torch.int32).cuda()
    l0 = cu.LAUNCHES
    pre, dec = _generate_timed(llm, prompts, o, args.steps, args.warmup)
    ms = pre + dec
    return {"metric": "output tok/s, Nemotron-H-style hybrid (Mamba2 + gated DeltaNet + GQA attention), bf16",
            "value": round(b * o / (ms / 1e3), 1), "unit": "tok/s", "n_gpus": 1, "ms_per_step": round(ms, 3),
            "config": {"global_batch": b, "seq_len": s, "output_len": o, "prefill_ms": round(pre, 3),
                       "decode_ms_per_token": round(dec / max(1, o - 1), 4), "layers": cfg.num_hidden_layers,
                       "layer_types": {t: cfg.layer_types.count(t) for t in sorted(set(cfg.layer_types))}},
            "gpu_launches": int(cu.LAUNCHES - l0), "data": "synthetic"}


def run_eagle(args) -> dict:
    from ..config import qwen3_8b_config
    from ..model import AutoModel
    from ..ops import cuda as cu
    from ..runtime.kv_cache import KVCacheManager
    from ..runtime.runner import ModelRunner
    from ..runtime.speculative import EagleDecoder, SpecConfig
    b, s, rounds = args.batch or 4, args.input_len or 2048, args.output_len or 32
    dev = torch.device("cuda", 0)
    kw = {"num_hidden_layers": args.layers} if args.layers else {}
    cfg = qwen3_8b_config(dtype="bfloat16", **kw)
    model = AutoModel.from_config(cfg, device=dev, random_init=0)
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
    emitted0, r0 = dec.stats.emitted, dec.stats.rounds
    e0, e1 = _events(2)
    e0.record()
    for _ in range(rounds):
        dec.round(seats)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    emitted = dec.stats.emitted - emitted0
    return {"metric": "output tok/s, EAGLE-3 tree speculative decoding on the Qwen3-8B shape (bf16), top-k 10, depth 6, 60 verify tokens",
            "value": round(emitted / (ms / 1e3), 1), "unit": "tok/s", "n_gpus": 1, "ms_per_round": round(ms / rounds, 3),
            "config": {"global_batch": b, "prompt_len": s, "rounds": rounds, "mean_accept_length": round(emitted / (rounds * b), 3),
                       "forced_accept_mean": 3.5, "prefill_s": round(t1 - t0, 3), "draft_forwards_per_round": spec.draft_steps,
                       "layers": cfg.num_hidden_layers, "note": "eager rounds (one device→host read per round); accept lengths are prescribed"},
            "gpu_launches": int(cu.LAUNCHES - l0), "data": "synthetic"}


def main(args) -> int:
    fn = {"moe": run_moe, "hybrid": run_hybrid, "eagle": run_eagle}[args.workload]
    out = fn(args)
    rank, world, llm = out.pop("_rank", 0), out.pop("_world", 1), out.pop("_llm", None)
    out.update({"steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "dtype": "bf16" if args.workload != "moe" else "nvfp4-experts/bf16"})
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
