"""Worker run under torch.distributed.run by the tensor-parallel tests (one process per rank).

Builds the same small decoder at TP=1 (rank-local reference) and TP=world, feeds identical
prompts and compares logits / greedy tokens.  Exits non-zero on mismatch."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    backend, kind, ckpt = sys.argv[1], sys.argv[2], sys.argv[3]
    prompt_len = int(sys.argv[4]) if len(sys.argv) > 4 else 70
    expert_parallel = len(sys.argv) > 5 and sys.argv[5] == "ep"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    from tensorrt_edge_llm_b200 import AutoModel
    from tensorrt_edge_llm_b200.config import Mapping
    from tensorrt_edge_llm_b200.parallel import make_comm
    from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
    from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

    def run(mapping, comm):
        model = AutoModel.from_pretrained(ckpt, mapping=mapping, comm=comm, device=dev)
        kv = KVCacheManager(model.cfg, num_pages=24, page_size=64, max_seats=4, max_pages_per_seq=6, device=dev)
        r = ModelRunner(model, kv, dev)
        g = torch.Generator().manual_seed(3)
        prompts = torch.randint(0, model.cfg.vocab_size, (2, prompt_len), generator=g).tolist()
        logits = r.prefill([0, 1], prompts)
        first = logits.float().argmax(-1).to(torch.int32)
        toks = r.decode_greedy([0, 1], first, 6)
        # sampled decode: with a vocabulary-sharded head the ranks exchange per-shard candidates instead of the logits
        from tensorrt_edge_llm_b200.runtime.runner import SamplingParams
        sp = SamplingParams(temperature=0.8, top_k=20, seed=7)
        kc = r._candidate_k(sp)
        sampled = r.decode_sampled([0, 1], toks[:, -1], 5, sp)
        sp2 = SamplingParams(temperature=0.7, top_p=0.9, seed=9)
        sampled2 = r.decode_sampled([0, 1], sampled[:, -1], 4, sp2)
        return logits.float().cpu(), toks.cpu(), torch.cat([sampled, sampled2], 1).cpu(), kc

    ref_logits, ref_toks, ref_sampled, _ = run(None, None)
    comm = make_comm(kind, dev)
    # vocabulary-sharded greedy pick: candidates per shard instead of gathered logits, ties across shards → lowest id
    g = torch.Generator().manual_seed(11)
    full = torch.randn(7, 40 * world, generator=g)
    full[0, 3] = full[0, 40 * world - 1] = 9.0
    full[1, 40 * world - 2] = 8.0
    full[2, 41 % (40 * world)] = full[2, 39] = 7.5
    want_ids = (full == full.max(-1, keepdim=True).values).to(torch.int32).argmax(-1).to(torch.int32)
    for dt in ((torch.float32, torch.bfloat16) if backend == "nccl" else (torch.float32,)):
        shard = full.to(dt)[:, rank * 40:(rank + 1) * 40].contiguous().to(dev)
        for _ in range(3):                   # epochs advance, tables alternate
            got_ids = comm.argmax_sharded(shard).cpu()
        want_dt = (full.to(dt).float() == full.to(dt).float().max(-1, keepdim=True).values).to(torch.int32).argmax(-1).to(torch.int32)
        if not torch.equal(got_ids, want_dt):
            print(f"rank {rank}: sharded arg-max {got_ids.tolist()} != {want_dt.tolist()} ({dt})", flush=True)
            sys.exit(1)
    del want_ids
    mapping = Mapping(tp_size=world, tp_rank=rank, ep_size=world if expert_parallel else 1, ep_rank=rank if expert_parallel else 0)
    tp_logits, tp_toks, tp_sampled, kc = run(mapping, comm)
    sampled_same = (tp_sampled == ref_sampled).float().mean().item()
    if world > 1 and kc != 20:
        print(f"rank {rank}: sampled decoding did not take the candidate exchange (k = {kc})", flush=True)
        sys.exit(1)
    if (dev.type == "cpu" and sampled_same < 1.0) or sampled_same < 0.4:
        print(f"rank {rank}: sampled tokens {tp_sampled.tolist()} != {ref_sampled.tolist()}", flush=True)
        sys.exit(1)
    err = (tp_logits - ref_logits).abs().max().item()
    scale = ref_logits.abs().max().item()
    tol = 1e-4 if dev.type == "cpu" else 0.06
    ok = err <= tol * max(scale, 1.0)
    same = (tp_toks == ref_toks).float().mean().item()
    if kind == "fused" and 2 * prompt_len > 256 and world > 1 and not comm._rs:
        print(f"rank {rank}: the reduce-scatter path was not taken", flush=True)
        ok = False
    if kind == "fused" and expert_parallel and 2 * prompt_len > 256 and world > 1 and not comm._ep:
        print(f"rank {rank}: the expert all-to-all path was not taken", flush=True)
        ok = False
    gathered = [None] * world
    dist.all_gather_object(gathered, tp_toks.tolist())
    identical = all(g == gathered[0] for g in gathered)
    # cross-rank view: every rank must hold the same TP logits, and the rank-local references must agree too
    both = [None] * world
    dist.all_gather_object(both, (tp_logits, ref_logits))
    tp_spread = max((b[0] - both[0][0]).abs().max().item() for b in both)
    ref_spread = max((b[1] - both[0][1]).abs().max().item() for b in both)
    per_seq = (tp_logits - ref_logits).abs().amax(-1).tolist()
    print(f"rank {rank}: per-sequence err {per_seq} tp spread over ranks {tp_spread:.3e} ref spread over ranks {ref_spread:.3e}", flush=True)
    if tp_spread > 0:
        ok = False
    if dev.type == "cuda":
        from tensorrt_edge_llm_b200.ops import cuda as cu
        torch.cuda.synchronize()
        cu.Workspace.get(dev).check_status()
    print(f"rank {rank}: max logit err {err:.3e} (scale {scale:.2f}) token agreement {same:.2f} ranks identical {identical}", flush=True)
    dist.barrier()
    bad = not ok or not identical or (dev.type == "cpu" and same < 1.0) or same < 0.5
    if dev.type == "cuda":
        # graphs captured with NCCL kernels are still alive: skip the collective destructor
        sys.stdout.flush()
        os._exit(1 if bad else 0)
    dist.destroy_process_group()
    if bad:
        sys.exit(1)


if __name__ == "__main__":
    main()
