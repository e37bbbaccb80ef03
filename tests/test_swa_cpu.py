"""Bounded sliding-window KV storage: pages behind the window go back to the pool and the outputs do not change."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def _cfg():
    return tiny_llama_config(num_hidden_layers=2, sliding_window=40, vocab_size=512)


def test_retire_boundary_and_page_accounting():
    cfg = _cfg()
    kv = KVCacheManager(cfg, num_pages=40, page_size=16, max_seats=2, max_pages_per_seq=40)
    assert kv.bounded_swa and kv.first_live_token(100) == 0 and kv.first_live_token(167) == 128 and kv.first_live_token(300) == 256
    kv.reserve(0, 300)
    assert kv.alloc.free_pages() == 40 - 19 if kv.native is None else kv.native.free_pages == 40 - 19
    kv.commit(0, 300)                                            # tokens below 256 are out of reach for every later query
    assert kv.live_pages(0) == 19 - 16 and kv.retired_pages == 16
    assert kv.table[0, :16].eq(-1).all() and kv.table[0, 16:19].ge(0).all()
    kv.reserve(0, 340)                                           # growth appends logical pages after the retired ones
    assert kv.live_pages(0) == 6 and len(kv.pages_of(0)) == 22
    kv.free(0)
    free = kv.native.free_pages if kv.native is not None else kv.alloc.free_pages()
    assert free == 40 and kv.live_pages(0) == 0
    assert not KVCacheManager(cfg, 8, 16, 2, 8, bounded_swa=False).bounded_swa
    assert not KVCacheManager(tiny_llama_config(), 8, 16, 2, 8).bounded_swa      # no window, nothing to bound


def test_outputs_match_unbounded_storage_and_pool_stays_small():
    cfg = _cfg()
    model = AutoModel.from_config(cfg, random_init=0)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab_size, (200,), generator=g).tolist()

    def run(bounded, pages):
        kv = KVCacheManager(cfg, num_pages=pages, page_size=16, max_seats=1, max_pages_per_seq=64, bounded_swa=bounded)
        r = ModelRunner(model, kv, max_num_tokens=64)            # the prompt runs as four chunks
        logits = r.prefill([0], [prompt])
        toks = [int(logits.argmax(-1))]
        peak = kv.live_pages(0)
        for _ in range(150):
            kv.reserve(0, kv.lengths[0] + 1)
            toks.append(int(r.step([0], [[toks[-1]]]).argmax(-1)))
            peak = max(peak, kv.live_pages(0))
        return toks, peak, kv

    ref_toks, ref_peak, _ = run(False, 64)
    toks, peak, kv = run(True, 64)
    assert toks == ref_toks
    assert ref_peak == 22 and peak <= kv.swa_live_pages_bound(64) and kv.retired_pages >= 16


def test_in_flight_batching_on_a_pool_smaller_than_the_sequences():
    """Three requests of 430 tokens each need 81 pages of full storage; 48 pages suffice when the window bounds them."""
    cfg = _cfg()
    full = LLM(cfg, device="cpu", max_batch_size=3, max_input_len=256, max_kv_cache_capacity=448, page_size=16, max_num_tokens=64,
               enable_in_flight_batching=True)
    full.kv.bounded_swa = False
    g = torch.Generator().manual_seed(9)
    prompts = torch.randint(0, cfg.vocab_size, (3, 180), generator=g).tolist()
    sp = SamplingParams(max_tokens=250, temperature=0.0, ignore_eos=True)
    want = [o.token_ids for o in full.generate(prompts, sp)]
    full.close()
    small = LLM(cfg, device="cpu", max_batch_size=3, max_input_len=256, max_kv_cache_capacity=448, page_size=16, max_num_tokens=64,
                enable_in_flight_batching=True, kv_pages=48)
    assert small.kv.bounded_swa and 3 * small.kv.swa_live_pages_bound(64) <= 48
    got = [o.token_ids for o in small.generate(prompts, sp)]
    assert got == want and small.kv.retired_pages > 0
    small.close()
