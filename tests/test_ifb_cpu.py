"""In-flight batching through the native request engine over the real model runner (CPU):
tokens must equal the static-batch run of the same prompts, whatever the batch composition."""
import torch

from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.llm import LLM
from tensorrt_edge_llm_b200.runtime.runner import SamplingParams


def _prompts():
    g = torch.Generator().manual_seed(5)
    return [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (5, 70, 131, 33, 9)]


def test_ifb_matches_static_batch_and_reuses_prefix():
    cfg = tiny_llama_config()
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    static = LLM(cfg, device="cpu", max_batch_size=8, max_input_len=256, max_kv_cache_capacity=320)
    want = [o.token_ids for o in static.generate(_prompts(), sp)]
    ifb = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=256, max_kv_cache_capacity=320,
              enable_in_flight_batching=True, enable_prefix_cache=True,
              scheduling={"mode": "mixed", "max_num_tokens": 128, "max_chunk_tokens": 64})
    outs = ifb.generate(_prompts(), sp)
    assert [o.token_ids for o in outs] == want
    m = ifb.engine.metrics()
    assert m.completed == 5 and m.admitted_mid_flight >= 1 and m.mixed_steps >= 1
    # the same long prompt again: its full pages come from the prefix cache
    again = ifb.generate([_prompts()[2]], sp)
    assert again[0].token_ids == want[2]
    assert ifb.engine.metrics().prefix_reused_tokens >= 128
    assert ifb.get_context_cache_counters()["reused_tokens"] >= 128 and ifb.get_scheduling_metrics()["completed"] == 6
    assert static.get_scheduling_metrics() is None and static.get_context_cache_counters() is None
    # streaming yields the same tokens
    streamed = []
    for toks, _ in ifb.generate_stream(_prompts()[1], sp):
        streamed += toks
    assert streamed == want[1]
    # sampling is reproducible per request regardless of what else is in the batch
    sps = SamplingParams(max_tokens=5, temperature=0.8, top_k=20, top_p=0.9, seed=7, ignore_eos=True)
    a = ifb.generate([_prompts()[0]], sps)[0].token_ids
    ifb.close()
    static.close()
    assert len(a) == 5


def test_context_cache_policies_per_request():
    cfg = tiny_llama_config()
    llm = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=256, max_kv_cache_capacity=384,
              enable_in_flight_batching=True, enable_prefix_cache=True)
    prompt = _prompts()[2]                                      # 131 tokens = two full 64-token pages
    sp = SamplingParams(max_tokens=70, ignore_eos=True)
    first = llm.generate([prompt], SamplingParams(max_tokens=70, ignore_eos=True, context_cache_commit="none"))[0]
    assert first.reused_input_tokens == 0
    again = llm.generate([prompt], sp)[0]                       # nothing was published by the first request
    assert again.reused_input_tokens == 0 and again.token_ids == first.token_ids
    third = llm.generate([prompt], SamplingParams(max_tokens=70, ignore_eos=True, context_cache_lookup=False,
                                                  context_cache_commit="including_generated_tokens"))[0]
    assert third.reused_input_tokens == 0                       # bypassed the lookup although the prompt pages exist now
    # a follow-up turn that quotes prompt + answer reuses the pages of both (201 tokens → three full pages)
    turn2 = prompt + third.token_ids + [11, 12, 13]
    out = llm.generate([turn2], SamplingParams(max_tokens=4, ignore_eos=True))[0]
    assert out.reused_input_tokens == 192
    import pytest
    with pytest.raises(ValueError):
        llm.generate([prompt], SamplingParams(max_tokens=2, context_cache_commit="sometimes"))
    llm.close()
