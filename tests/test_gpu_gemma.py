"""Gemma 3 text decoder (256-wide heads, sliding and full attention layers) on the GPU kernels against the same weights on the CPU."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import ModelConfig
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

pytestmark = pytest.mark.gpu


def test_gemma3_head_dim_256_prefill_and_decode_match_cpu():
    hf = dict(model_type="gemma3_text", vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
              num_key_value_heads=2, head_dim=256, sliding_window=96, query_pre_attn_scalar=256, max_position_embeddings=1024,
              layer_types=["sliding_attention", "full_attention", "sliding_attention"], dtype="bfloat16")
    cfg = ModelConfig.from_hf_dict(hf)
    assert cfg.head_dim == 256
    dev = torch.device("cuda", 0)
    gpu = AutoModel.from_config(cfg, device=dev, random_init=0)
    cpu = AutoModel.from_config(cfg, random_init=0)
    cpu.load_state_dict({k: v.cpu() for k, v in gpu.state_dict().items()})
    cpu = cpu.float()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (200, 37)]

    def run(model, device):
        kv = KVCacheManager(model.cfg, num_pages=16, page_size=64, max_seats=2, max_pages_per_seq=6, device=device,
                            **({"dtype": torch.float32} if device.type == "cpu" else {}))
        r = ModelRunner(model, kv)
        r.use_cuda_graphs = False
        out = [r.prefill([0, 1], prompts).float().cpu()]
        toks = [[5], [9]]
        for _ in range(3):                      # decode rows attend through the tile kernel (the decode kernel takes 128-wide heads)
            out.append(r.step([0, 1], toks).float().cpu())
            toks = [[int(t)] for t in out[-1].argmax(-1)]
        return out

    got = run(gpu, dev)
    want = run(cpu, torch.device("cpu"))
    for a, b in zip(got, want):
        err = (a - b).norm() / b.norm()
        assert err < 3e-2, float(err)
