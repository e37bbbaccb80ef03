"""Multimodal RoPE on the GPU path: the rope kernel reads the per-row tables the model prepares."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

pytestmark = pytest.mark.gpu


def test_mrope_gpu_matches_cpu():
    cfg = tiny_llama_config(num_hidden_layers=2, vocab_size=512, dtype="bfloat16", hidden_size=512, num_attention_heads=4,
                            num_key_value_heads=2, head_dim=128)
    cfg.mrope_section = [16, 24, 24]
    cpu = AutoModel.from_config(cfg, random_init=0)
    gpu = AutoModel.from_config(cfg, device=torch.device("cuda", 0), random_init=0)
    ids = [3, 4] + [9] * 24 + list(range(20, 60))
    pos3, delta = ref.mrope_positions(ids, 9, [(1, 8, 12)])
    outs = []
    for model, dev in ((cpu, "cpu"), (gpu, "cuda")):
        kv = KVCacheManager(cfg, num_pages=8, page_size=64, max_seats=1, max_pages_per_seq=4, device=dev)
        r = ModelRunner(model, kv)
        logits = r.prefill_embeds([0], [r.embed_tokens(ids)], positions3=[pos3], rope_deltas=[delta])
        nxt = r.step([0], [[int(logits.float().argmax(-1))]])
        outs.append((logits.float().cpu(), nxt.float().cpu()))
    for a, b in zip(outs[0], outs[1]):
        assert (a - b).abs().max() < 0.06 * max(a.abs().max().item(), 1.0)
    # and the positions matter: ordinary positions give different logits on the GPU too
    kv = KVCacheManager(cfg, num_pages=8, page_size=64, max_seats=1, max_pages_per_seq=4, device="cuda")
    r = ModelRunner(gpu, kv)
    plain = r.prefill([0], [ids]).float().cpu()
    assert (plain - outs[1][0]).abs().max() > 1e-2
