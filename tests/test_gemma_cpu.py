"""Gemma 3 text decoder against Hugging Face ``Gemma3ForCausalLM`` (same random checkpoint), prefill and decode."""
import json
import os

import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.checkpoint import save_file
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def test_matches_hf_gemma3(tmp_path):
    from transformers import Gemma3ForCausalLM, Gemma3TextConfig
    hc = Gemma3TextConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=16, sliding_window=8, query_pre_attn_scalar=24, max_position_embeddings=256,
                          layer_types=["sliding_attention", "sliding_attention", "full_attention", "sliding_attention"],
                          attn_implementation="eager", dtype="float32")
    torch.manual_seed(0)
    hf = Gemma3ForCausalLM(hc).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.copy_(torch.randn_like(p) * 0.2)            # stored as w - 1: make the +1 folding matter
    d = str(tmp_path)
    save_file({k: v.contiguous() for k, v in hf.state_dict().items() if k != "lm_head.weight"}, os.path.join(d, "model.safetensors"))
    json.dump(hc.to_dict(), open(os.path.join(d, "config.json"), "w"))
    model = AutoModel.from_pretrained(d)
    cfg = model.cfg
    assert type(model).__name__ == "GemmaCausalLM" and cfg.layer_windows == [8, 8, 0, 8] and cfg.rope_local_theta == 10000.0
    assert cfg.rope_theta == 1e6 and cfg.query_pre_attn_scalar == 24 and cfg.hidden_act == "gelu_pytorch_tanh"
    kv = KVCacheManager(cfg, num_pages=16, page_size=16, max_seats=2, max_pages_per_seq=8)
    assert not kv.bounded_swa                                  # a full-attention layer keeps the whole history
    r = ModelRunner(model, kv)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 300, (1, 40), generator=g)
    with torch.no_grad():
        want = hf(ids).logits[0]
    got = r.prefill([0], [ids[0].tolist()])
    assert (got[0] - want[-1]).abs().max() < 2e-4 * max(1.0, want.abs().max().item())
    # decode continues past the window: greedy tokens agree with a full Hugging Face pass each step
    seq = ids[0].tolist()
    tok = int(got[0].argmax())
    for _ in range(6):
        seq.append(tok)
        with torch.no_grad():
            ref_next = int(hf(torch.tensor([seq])).logits[0, -1].argmax())
        tok = int(r.step([0], [[tok]])[0].argmax())
        assert tok == ref_next


def test_embedding_rows_fed_directly_match_token_ids():
    """Prompts fed as embedding rows (multimodal path) see the same scaled rows as prompts fed as ids."""
    from tensorrt_edge_llm_b200.config import ModelConfig
    hf = dict(model_type="gemma3_text", vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=8, sliding_window=0, layer_types=["full_attention"] * 2, max_position_embeddings=128, dtype="float32")
    cfg = ModelConfig.from_hf_dict(hf)
    model = AutoModel.from_config(cfg, random_init=0)               # random init keeps the sqrt(hidden) multiplier outside the table
    assert model.model.embed_scale != 1.0
    kv = KVCacheManager(cfg, num_pages=8, page_size=16, max_seats=2, max_pages_per_seq=4)
    r = ModelRunner(model, kv)
    ids = [5, 9, 33, 2, 77, 12]
    a = r.prefill([0], [ids])
    b = r.prefill_embeds([1], [r.embed_tokens(ids)])
    assert (a - b).abs().max() < 1e-5
