"""Qwen3-MoE decoder on CPU against the Hugging Face implementation, plus expert-parallel sharding."""
import json
import os

import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.checkpoint import save_file
from tensorrt_edge_llm_b200.config import Mapping
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM
    cfg = Qwen3MoeConfig(vocab_size=1000, hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=8, num_experts_per_tok=2,
                         norm_topk_prob=True, rms_norm_eps=1e-6, rope_theta=1e4, max_position_embeddings=512,
                         decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False, output_router_logits=False)
    torch.manual_seed(0)
    m = Qwen3MoeForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" not in n:
                p.normal_(0.0, 0.05)
    d = tmp_path_factory.mktemp("moe")
    sd = {}
    for k, v in m.state_dict().items():
        if k.endswith("experts.gate_up_proj"):         # fused expert tensors [E, 2I, H] → per-expert HF names
            base = k[:-len(".gate_up_proj")]
            for e in range(v.shape[0]):
                i = v.shape[1] // 2
                sd[f"{base}.{e}.gate_proj.weight"] = v[e, :i].contiguous()
                sd[f"{base}.{e}.up_proj.weight"] = v[e, i:].contiguous()
        elif k.endswith("experts.down_proj"):
            base = k[:-len(".down_proj")]
            for e in range(v.shape[0]):
                sd[f"{base}.{e}.down_proj.weight"] = v[e].contiguous()
        else:
            sd[k] = v
    save_file(sd, os.path.join(d, "model.safetensors"))
    hf = cfg.to_dict()
    hf["torch_dtype"] = "float32"
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    return str(d), m


def _run(model, prompts):
    kv = KVCacheManager(model.cfg, num_pages=16, page_size=64, max_seats=4, max_pages_per_seq=4)
    r = ModelRunner(model, kv)
    return r.prefill([0, 1], prompts)


def test_moe_matches_hf(ckpt):
    d, hf = ckpt
    model = AutoModel.from_pretrained(d)
    assert model.cfg.num_experts == 8 and type(model).__name__ == "MoECausalLM"
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, 1000, (2, 40), generator=g)
    logits = _run(model, prompts.tolist())
    with torch.no_grad():
        want = hf(prompts).logits[:, -1]
    assert (logits - want).abs().max() < 2e-4


def test_expert_parallel_partial_sums_add_up(ckpt):
    d, _ = ckpt
    full = AutoModel.from_pretrained(d)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, 128, generator=g)
    want = full.model.layers[0].mlp(x)
    parts = []
    for r in range(4):
        m = AutoModel.from_pretrained(d, mapping=Mapping(tp_size=1, tp_rank=0, ep_size=4, ep_rank=r))
        parts.append(m.model.layers[0].mlp(x))
    assert (sum(parts) - want).abs().max() < 1e-5
    tparts = []
    for r in range(2):
        m = AutoModel.from_pretrained(d, mapping=Mapping(tp_size=2, tp_rank=r))
        tparts.append(m.model.layers[0].mlp(x))
    assert (sum(tparts) - want).abs().max() < 1e-5


def test_shared_expert_matches_hf(tmp_path):
    """Qwen2-MoE: routed experts plus a shared expert scaled by sigmoid(shared_expert_gate · x), against Hugging Face."""
    from transformers import Qwen2MoeConfig, Qwen2MoeForCausalLM
    cfg = Qwen2MoeConfig(vocab_size=1000, hidden_size=128, intermediate_size=256, moe_intermediate_size=64, shared_expert_intermediate_size=96,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, num_experts=8, num_experts_per_tok=2,
                         norm_topk_prob=False, rms_norm_eps=1e-6, rope_theta=1e4, max_position_embeddings=512, decoder_sparse_step=1,
                         mlp_only_layers=[], tie_word_embeddings=False, output_router_logits=False, use_sliding_window=False)
    torch.manual_seed(0)
    m = Qwen2MoeForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" not in n:
                p.normal_(0.0, 0.05)
    sd = {}
    for k, v in m.state_dict().items():
        if k.endswith("experts.gate_up_proj"):
            base, i = k[:-len(".gate_up_proj")], v.shape[1] // 2
            for e in range(v.shape[0]):
                sd[f"{base}.{e}.gate_proj.weight"], sd[f"{base}.{e}.up_proj.weight"] = v[e, :i].contiguous(), v[e, i:].contiguous()
        elif k.endswith("experts.down_proj"):
            for e in range(v.shape[0]):
                sd[f"{k[:-len('.down_proj')]}.{e}.down_proj.weight"] = v[e].contiguous()
        else:
            sd[k] = v
    save_file(sd, os.path.join(tmp_path, "model.safetensors"))
    hf = cfg.to_dict()
    hf["torch_dtype"] = "float32"
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(hf, f)
    model = AutoModel.from_pretrained(str(tmp_path))
    blk = model.model.layers[0].mlp
    assert blk.shared_expert is not None and blk.shared_expert_gate.weight.shape == (1, 128)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, 1000, (2, 40), generator=g)
    logits = _run(model, prompts.tolist())
    with torch.no_grad():
        want = m(prompts).logits[:, -1]
    assert (logits - want).abs().max() < 2e-4
    # tensor-parallel partial sums of the whole block (routed + shared) add up
    x = torch.randn(7, 128, generator=g)
    full = blk(x)
    parts = [AutoModel.from_pretrained(str(tmp_path), mapping=Mapping(tp_size=2, tp_rank=r)).model.layers[0].mlp(x) for r in range(2)]
    assert (sum(parts) - full).abs().max() < 1e-5
