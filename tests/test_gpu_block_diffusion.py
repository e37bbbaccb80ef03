"""Block diffusion on the GPU path: the canvas pass (tree-mask attention with every bit set, several mask words) against
the CPU reference ops, and the decoder end to end."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import ModelConfig
from tensorrt_edge_llm_b200.runtime import block_diffusion as bd
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

pytestmark = pytest.mark.gpu


def _cfg(canvas):
    hf = dict(model_type="diffusion_gemma", vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, sliding_window=0, layer_types=["full_attention"] * 2,
              max_position_embeddings=1024, dtype="bfloat16", diffusion=dict(canvas_length=canvas, max_denoising_steps=3))
    return ModelConfig.from_hf_dict(hf)


def test_canvas_pass_gpu_matches_cpu():
    canvas_len = 72                                       # three mask words, the last one partly used
    cfg = _cfg(canvas_len)
    prompt = [(7 * i + 3) % 512 for i in range(50)]
    canvas = torch.tensor([(13 * i + 5) % 512 for i in range(canvas_len)])
    outs = []
    for dev in ("cpu", "cuda"):
        model = AutoModel.from_config(cfg, device=torch.device(dev), random_init=0)
        kv = KVCacheManager(cfg, num_pages=8, page_size=64, max_seats=1, max_pages_per_seq=4, device=dev)
        r = ModelRunner(model, kv)
        r.prefill([0], [prompt])
        soft = model.soft_embeddings(torch.linspace(-2, 2, canvas_len * 512).reshape(canvas_len, 512).to(dev), 0.6)
        x = model.canvas_inputs(canvas.to(dev), soft)
        meta = r._meta([0], [canvas_len], logits_all=True, tree_mask=bd.full_mask(canvas_len, canvas_len, dev))
        outs.append(model(None, meta, r.cache, inputs_embeds=x).float().cpu())
        assert kv.lengths[0] == len(prompt)
    assert (outs[0] - outs[1]).abs().max() < 0.06 * max(outs[0].abs().max().item(), 1.0)


def test_decoder_runs_on_gpu():
    cfg = _cfg(64)
    model = AutoModel.from_config(cfg, device=torch.device("cuda", 0), random_init=0)
    kv = KVCacheManager(cfg, num_pages=16, page_size=64, max_seats=2, max_pages_per_seq=6, device="cuda")
    r = ModelRunner(model, kv)
    dec = bd.BlockDiffusionDecoder(r)
    prompts = [[1, 2, 3, 4, 5, 6], [9, 8, 7]]
    out = dec.generate([0, 1], prompts, max_tokens=100, eos_ids=[])
    assert [len(o) for o in out] == [100, 100] and kv.lengths[0] == 106 and kv.lengths[1] == 103
    assert dec.stats.blocks == 2 and 2 <= dec.stats.denoise_passes <= 6
    # the cache the commit passes wrote is the causal cache of prompt + output
    probe = r.step([0], [[out[0][-1]]], commit=False).float().cpu()
    kv2 = KVCacheManager(cfg, num_pages=8, page_size=64, max_seats=1, max_pages_per_seq=6, device="cuda")
    ref = ModelRunner(model, kv2).prefill([0], [prompts[0] + out[0] + [out[0][-1]]]).float().cpu()
    assert (probe - ref).abs().max() < 0.06 * max(ref.abs().max().item(), 1.0)
