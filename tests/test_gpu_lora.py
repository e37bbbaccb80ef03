"""LoRA on the GPU path: a single adapter and a step that mixes adapters (stacked factors) against the CPU reference ops."""
import json
import os

import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.checkpoint import save_file
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.lora.runtime import LoraLinear, LoraManager
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

pytestmark = pytest.mark.gpu


def _adapter_dir(d, seed, rank, hidden, inter):
    os.makedirs(d, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    mods = {"model.layers.0.self_attn.q_proj": (hidden, hidden), "model.layers.0.self_attn.v_proj": (256, hidden),
            "model.layers.1.mlp.down_proj": (hidden, inter)}
    t = {}
    for mod, (o, i) in mods.items():
        t[f"lora_A_{mod}"] = (torch.randn(rank, i, generator=g) * 0.05).to(torch.bfloat16)
        t[f"lora_B_{mod}"] = (torch.randn(o, rank, generator=g) * 0.3).to(torch.bfloat16)
    save_file(t, os.path.join(d, "lora_weights.safetensors"))
    with open(os.path.join(d, "lora_config.json"), "w") as f:
        json.dump({"rank": rank, "scale_folded_into_B": True, "modules": sorted(mods)}, f)


def test_lora_single_and_mixed_adapters_gpu_match_cpu(tmp_path):
    cfg = tiny_llama_config(num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=128, vocab_size=1000, dtype="bfloat16")
    d1, d2 = str(tmp_path / "a1"), str(tmp_path / "a2")
    _adapter_dir(d1, 1, 8, 512, 1024)
    _adapter_dir(d2, 2, 4, 512, 1024)
    model = AutoModel.from_config(cfg, random_init=0)
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    prompts = [[(7 * i + 3) % 990 for i in range(20)], [(5 * i + 1) % 990 for i in range(33)], [(3 * i + 2) % 990 for i in range(12)]]

    def run(device):
        m = AutoModel.from_config(cfg)
        m.load_state_dict(sd)
        m = m.to(device)
        mgr = LoraManager(m)
        mgr.load_adapter("one", d1)
        mgr.load_adapter("two", d2)
        r = ModelRunner(m, KVCacheManager(cfg, num_pages=8, page_size=64, max_seats=3, max_pages_per_seq=2, device=device), device)
        r.use_cuda_graphs = False
        r.lora = mgr
        outs = []
        mgr.set_active("one")
        outs.append(r.prefill([0], [prompts[0]]).float().cpu())
        r.kv.free(0)
        mgr.set_active(None)
        # one step, three sequences, three routes: adapter one, no adapter, adapter two
        n0, n1, n2 = (len(p) for p in prompts)
        mgr.set_segments([(0, n0, "one"), (n0, n0 + n1, None), (n0 + n1, n0 + n1 + n2, "two")])
        outs.append(r.prefill([0, 1, 2], prompts).float().cpu())
        mgr.set_segments(None)
        return outs

    calls0 = LoraLinear.grouped_calls
    gpu = run(torch.device("cuda", 0))
    assert LoraLinear.grouped_calls > calls0
    cpu = run(torch.device("cpu"))
    for x, y in zip(gpu, cpu):
        assert x.shape == y.shape
        assert (x - y).abs().max() < 0.06 * max(y.abs().max().item(), 1.0)
    # the adapters matter: routed rows differ from the base model's
    base = AutoModel.from_config(cfg)
    base.load_state_dict(sd)
    r = ModelRunner(base, KVCacheManager(cfg, num_pages=8, page_size=64, max_seats=3, max_pages_per_seq=2))
    plain = r.prefill([0, 1, 2], prompts).float()
    assert (plain[0] - cpu[1][0]).abs().max() > 5 * (gpu[1][0] - cpu[1][0]).abs().max()
    assert (plain[1] - cpu[1][1]).abs().max() < 1e-2 * max(plain.abs().max().item(), 1.0)
