"""Bounded sliding-window storage on the GPU kernels: retired (-1) page-table entries are never dereferenced."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

pytestmark = pytest.mark.gpu


def test_bounded_swa_matches_full_storage_on_gpu():
    dev = torch.device("cuda", 0)
    cfg = tiny_llama_config(num_hidden_layers=2, sliding_window=200, vocab_size=512, dtype="bfloat16", head_dim=128, num_attention_heads=4,
                            num_key_value_heads=2, hidden_size=512)
    model = AutoModel.from_config(cfg, device=dev, random_init=0)
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(0, cfg.vocab_size, (2, 700), generator=g).tolist()

    def run(bounded):
        kv = KVCacheManager(cfg, num_pages=40, page_size=64, max_seats=2, max_pages_per_seq=20, device=dev, bounded_swa=bounded)
        r = ModelRunner(model, kv, max_num_tokens=512)
        logits = r.prefill([0, 1], prompts)
        first = logits.float().argmax(-1).to(torch.int32)
        toks = r.decode_greedy([0, 1], first, 40)
        more = r.decode_greedy([0, 1], toks[:, -1].contiguous(), 40)       # second graph run sees the retired rows
        return logits.float().cpu(), torch.cat([toks, more], 1).cpu(), kv

    ref_logits, ref_toks, _ = run(False)
    logits, toks, kv = run(True)
    assert kv.retired_pages >= 2 * 7 and (kv.table[:2, :7] == -1).all()
    assert torch.equal(logits, ref_logits) and torch.equal(toks, ref_toks)
