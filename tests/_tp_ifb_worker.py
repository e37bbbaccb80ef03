"""Worker of the tensor-parallel in-flight-batching test: rank 0 runs the request engine, the others follow."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from tensorrt_edge_llm_b200.config import Mapping, tiny_llama_config
    from tensorrt_edge_llm_b200.parallel import make_comm
    from tensorrt_edge_llm_b200.parallel.tp_serving import StepMirror, serve_follower
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    ckpt = sys.argv[1]                                # every rank loads its shard of the same checkpoint
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (5, 70, 131, 33, 9)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    kw = dict(device="cpu", max_input_len=256, max_kv_cache_capacity=320, page_size=16)
    comm = make_comm("nccl", torch.device("cpu"))
    mirror = StepMirror()
    shard = Mapping(tp_size=world, tp_rank=rank)
    if rank == 0:
        single = LLM(ckpt, max_batch_size=8, **kw)
        want = [o.token_ids for o in single.generate(prompts, sp)]
        # a multimodal-style prompt: placeholder ids whose rows are replaced by "media" embedding rows
        mm_ids = [3, 4, 5] + [7] * 20 + [6, 8]
        mm_emb = single.runner.embed_tokens(mm_ids).clone()
        mm_emb[3:23] = (torch.randn(20, mm_emb.shape[1], generator=g) * 0.05).to(mm_emb.dtype)
        single.kv.free(0)
        single.kv.reserve(0, len(mm_ids) + 6)
        first = single.runner.pick(single.runner.prefill_embeds([0], [mm_emb]))
        want_mm = [int(first[0])] + single.runner.decode_greedy([0], first, 5)[0].tolist()
        single.close()
        llm = LLM(ckpt, mapping=shard, comm=comm, max_batch_size=2, enable_in_flight_batching=True, tp_mirror=mirror,
                  enable_prefix_cache=True, scheduling={"mode": "mixed", "max_num_tokens": 128, "max_chunk_tokens": 64}, **kw)
        got = [o.token_ids for o in llm.generate(prompts, sp)]
        # the long prompts again: their full pages come from the prefix index, on every rank alike
        again = [o.token_ids for o in llm.generate([prompts[2], prompts[1]], sp)]
        reused = llm.engine.metrics().prefix_reused_tokens
        m = llm.engine.metrics()
        # the embedding rows travel to the followers with the step (chunked: 25 rows at 16 per chunk)
        got_mm = [int(t) for t in llm.submit_multimodal(mm_ids, mm_emb, sp).get(600.0)]
        llm.close()                                   # tells the followers to stop
        ok = (got == want and m.completed == 7 and m.admitted_mid_flight >= 1 and got_mm == want_mm and again == [want[2], want[1]]
              and reused >= 128)
        print(f"rank 0: prefix reuse {reused} tokens, repeat match {again == [want[2], want[1]]}", flush=True)
        print(f"rank 0: multimodal match {got_mm == want_mm}", flush=True)
        print(f"rank 0: match {got == want}, completed {m.completed}, mid-flight admissions {m.admitted_mid_flight}, mirrored ops {mirror.sent}", flush=True)
    else:
        llm = LLM(ckpt, mapping=shard, comm=comm, max_batch_size=2, **kw)
        steps = serve_follower(llm.runner, mirror, enable_prefix_cache=True)
        ok = steps > 10
        print(f"rank {rank}: followed {steps} steps", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
