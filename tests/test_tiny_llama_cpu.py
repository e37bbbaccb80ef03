"""Plumbing check: the tiny Llama decoder stepped through the runtime's own code path (config,
loader, paged KV, ragged prefill, greedy decode) must match a Hugging Face forward to 1e-4."""
import json
import os

import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.checkpoint import save_file
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def _hf_model():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
                      rope_theta=1e4, max_position_embeddings=2048, tie_word_embeddings=False,
                      attention_bias=False, mlp_bias=False)
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" not in n:
                p.normal_(0.0, 0.02)
    return cfg, m


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    cfg, m = _hf_model()
    d = tmp_path_factory.mktemp("tiny_llama")
    save_file({k: v for k, v in m.state_dict().items()}, os.path.join(d, "model.safetensors"))
    hf = cfg.to_dict()
    hf["torch_dtype"] = "float32"
    hf["rope_theta"] = 1e4
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    return str(d), m


def test_config1_logits_match_hf(ckpt):
    d, hf = ckpt
    model = AutoModel.from_pretrained(d)
    assert model.cfg.dtype == "float32" and model.cfg.num_key_value_heads == 2
    kv = KVCacheManager(model.cfg, num_pages=16, page_size=64, max_seats=4, max_pages_per_seq=4)
    runner = ModelRunner(model, kv, max_num_tokens=160)        # forces a chunked second prompt
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, 32000, (2, 128), generator=g)
    seats = [0, 1]
    logits = runner.prefill(seats, [p.tolist() for p in prompts])
    seqs = prompts.clone()
    with torch.no_grad():
        ref = hf(seqs).logits[:, -1]
    assert (logits - ref).abs().max() < 1e-4
    toks = logits.argmax(-1)
    for step in range(32):
        seqs = torch.cat([seqs, toks[:, None]], dim=1)
        logits = runner.step(seats, [[int(t)] for t in toks])
        with torch.no_grad():
            ref = hf(seqs).logits[:, -1]
        err = (logits - ref).abs().max().item()
        assert err < 1e-4, f"step {step}: {err}"
        assert torch.equal(logits.argmax(-1), ref.argmax(-1))
        toks = logits.argmax(-1)
    assert kv.lengths[0] == 128 + 32


def test_decode_greedy_matches_stepwise(ckpt):
    d, _ = ckpt
    model = AutoModel.from_pretrained(d)
    kv = KVCacheManager(model.cfg, num_pages=16, page_size=64, max_seats=4, max_pages_per_seq=4)
    runner = ModelRunner(model, kv)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, 32000, (2, 40), generator=g)
    first = runner.prefill([0, 1], [p.tolist() for p in prompts]).argmax(-1).to(torch.int32)
    out = runner.decode_greedy([0, 1], first, 8)
    assert out.shape == (2, 8)
    kv2 = KVCacheManager(model.cfg, num_pages=16, page_size=64, max_seats=4, max_pages_per_seq=4)
    r2 = ModelRunner(model, kv2)
    t = r2.prefill([0, 1], [p.tolist() for p in prompts]).argmax(-1)
    for i in range(8):
        t = r2.step([0, 1], [[int(x)] for x in t]).argmax(-1)
        assert torch.equal(t.to(torch.int32), out[:, i])


def test_quantized_embedding_tables():
    import torch
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.models.embedding import QuantizedEmbedding
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    w = torch.randn(500, 64, generator=torch.Generator().manual_seed(0)) * 0.05
    ids = torch.tensor([3, 499, 0, 3], dtype=torch.int32)
    for fmt, tol, ratio in (("fp8", 0.07, 0.6), ("nvfp4", 0.2, 0.35)):
        q = QuantizedEmbedding.from_dense(w, fmt)
        got = q(ids)
        assert got.shape == (4, 64) and (got - w[ids.long()]).abs().max() < tol * w.abs().max()
        assert torch.equal(got[0], got[3]) and q.table_bytes() < ratio * w.numel() * 4
    cfg = tiny_llama_config(num_hidden_layers=2)
    prompts = [[5, 9, 33, 70], [8, 2, 44]]
    sp = SamplingParams(max_tokens=5)
    dense = LLM(cfg, device="cpu", max_batch_size=2, max_kv_cache_capacity=128)
    ref_logits = dense.runner.prefill([0], [prompts[0]]).float()
    dense.kv.free(0)
    q8 = LLM(cfg, device="cpu", max_batch_size=2, max_kv_cache_capacity=128, embedding_quantization="fp8")
    assert type(q8.model.model.embed_tokens).__name__ == "QuantizedEmbedding"
    lg = q8.runner.prefill([0], [prompts[0]]).float()
    q8.kv.free(0)
    cos = torch.nn.functional.cosine_similarity(lg.flatten(), ref_logits.flatten(), dim=0)
    assert float(cos) > 0.99 and len(q8.generate(prompts, sp)[1].token_ids) == 5
