"""InternVL vision tower + pixel-shuffle projector against Hugging Face ``InternVLModel.get_image_features``."""
import pytest
import torch

from tensorrt_edge_llm_b200.models.internvl_vision import InternVisionConfig, InternVisionEncoder


@pytest.mark.parametrize("variant", ["layer_norm", "rms_qk_norm"])
def test_matches_hf(variant):
    from transformers.models.internvl.configuration_internvl import InternVLConfig, InternVLVisionConfig
    from transformers.models.internvl.modeling_internvl import InternVLModel
    rms = variant == "rms_qk_norm"
    vc = InternVLVisionConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=96, image_size=[56, 56],
                              patch_size=[14, 14], attention_bias=rms, use_qk_norm=rms, norm_type="rms_norm" if rms else "layer_norm",
                              use_mean_pooling=not rms)
    text = dict(model_type="qwen2", vocab_size=100, hidden_size=48, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                num_key_value_heads=2)
    hc = InternVLConfig(vision_config=vc.to_dict(), text_config=text, downsample_ratio=0.5)
    hc._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = InternVLModel(hc).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "vision_tower" in n or "projector" in n:
                if "norm" in n or n.endswith("bias") or "lambda" in n or "cls_token" in n or "position_embeddings" in n:
                    p.copy_(torch.randn_like(p) * 0.3 + (1.0 if (n.endswith("weight") or "lambda" in n) else 0.0))
    full = hc.to_dict()
    cfg = InternVisionConfig.from_hf(full)
    cfg.dtype = "float32"
    assert (cfg.grid, cfg.out_hidden_size, cfg.use_qk_norm, cfg.rms_norm, cfg.final_layernorm) == (4, 48, rms, rms, rms)
    enc = InternVisionEncoder(cfg)
    assert enc.load_hf_state_dict(hf.state_dict()) == []
    px = torch.randn(3, 3, 56, 56, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf.get_image_features(px, vision_feature_layer=-1, vision_feature_select_strategy="default").pooler_output
    got = enc(px)
    assert got.shape == (3 * 4, 48) and want.shape == (3, 4, 48)
    assert (got - want.reshape(12, 48)).abs().max() < 2e-4 * max(1.0, want.abs().max().item())
    with pytest.raises(ValueError):
        enc(torch.zeros(1, 3, 42, 56))


def test_tile_grid_and_runner():
    import numpy as np
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.models.internvl_vision import tile_grid
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.multimodal import MultimodalInputs, MultimodalRunner
    assert tile_grid(448, 448, 448) == (1, 1) and tile_grid(1000, 500, 448) == (2, 1) and tile_grid(500, 1500, 448) == (1, 3)
    assert tile_grid(1600, 1200, 448, max_tiles=12) == (4, 3)
    cols, rows = tile_grid(1600, 1200, 448, max_tiles=6)
    assert cols * rows <= 6 and abs(cols / rows - 4 / 3) <= abs(1 - 4 / 3)
    cfg = tiny_llama_config(num_hidden_layers=2, vocab_size=200, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                            dtype="float32")
    llm = LLM(cfg, device="cpu", max_batch_size=1, max_input_len=256, max_kv_cache_capacity=320, page_size=16)
    vc = InternVisionConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, image_size=56, patch_size=14,
                            out_hidden_size=64, dtype="float32")
    tower = InternVisionEncoder(vc).random_init(0, std=0.1)
    mm = MultimodalRunner(llm, vision=tower, image_token_id=9, max_tiles=4)
    rng = np.random.default_rng(0)
    wide = rng.integers(0, 255, (50, 160, 3), dtype=np.uint8)                   # → 3 × 1 tiles + thumbnail
    square = rng.integers(0, 255, (60, 60, 3), dtype=np.uint8)                  # → one tile, no thumbnail
    rows = mm.encode_images([wide, square])
    assert rows[0].shape == (4 * 4, 64) and rows[1].shape == (4, 64)
    # the square image's rows equal a direct pass over its resized tile
    from tensorrt_edge_llm_b200.runtime import native as rt
    im = rt.resize_bicubic(rt.image_from_array(square), 56, 56)
    chw = torch.from_numpy(rt.normalize_chw(im, list(tower.image_mean), list(tower.image_std)))
    assert torch.allclose(rows[1], tower(chw[None]), atol=1e-5)
    out = mm.generate(MultimodalInputs().text([3, 4]).image(wide).text([5]), max_tokens=3)
    assert len(out) == 3
