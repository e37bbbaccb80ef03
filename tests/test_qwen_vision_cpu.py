"""Qwen2-VL / Qwen2.5-VL vision towers against the Hugging Face implementations (same random weights, fp32)."""
import pytest
import torch

from tensorrt_edge_llm_b200.models.qwen_vl_vision import (QwenVisionConfig, QwenVisionEncoder, patchify_frames, rotary_rows, window_order)

GRIDS = [(1, 6, 10), (2, 4, 4), (1, 2, 2)]


def _patches(cfg, grids, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(sum(t * h * w for t, h, w in grids), cfg.patch_dim, generator=g)


def test_qwen2_5_vl_window_attention_matches_hf():
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel
    hc = Qwen2_5_VLVisionConfig(depth=4, hidden_size=80, intermediate_size=96, num_heads=4, patch_size=14, spatial_merge_size=2,
                                temporal_patch_size=2, window_size=56, out_hidden_size=48, fullatt_block_indexes=[1, 3])
    hc._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = Qwen2_5_VisionTransformerPretrainedModel(hc).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or "ln_q" in n or n.endswith("bias"):
                p.copy_(torch.randn_like(p) * 0.3 + (1.0 if n.endswith("weight") else 0.0))
    cfg = QwenVisionConfig.from_hf(hc.to_dict())
    cfg.dtype = "float32"
    assert cfg.gated_mlp and cfg.window_size == 56 and cfg.head_dim == 20 and cfg.padded_head_dim == 64
    enc = QwenVisionEncoder(cfg)
    left = enc.load_hf_state_dict({"visual." + k: v for k, v in hf.state_dict().items()})
    assert left == []
    x = _patches(cfg, GRIDS)
    with torch.no_grad():
        want = hf(x, grid_thw=torch.tensor(GRIDS)).pooler_output
    got = enc(x, GRIDS)
    assert got.shape == want.shape == (sum(t * h * w for t, h, w in GRIDS) // 4, 48)
    assert (got - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item())
    # the window order is a permutation, windows at the edges are smaller, and every frame is covered
    order, lengths = window_order(GRIDS, 56, 2, 14)
    assert sorted(order.tolist()) == list(range(15 + 8 + 1)) and sum(lengths) == x.shape[0]
    assert lengths[:6] == [16, 16, 8, 8, 8, 4]              # 3 × 5 merged units in 2 × 2 windows: 2x2, 2x2, 2x1, 1x2, 1x2, 1x1 units


def test_qwen2_vl_full_attention_matches_hf():
    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig
    from transformers.models.qwen2_vl.modeling_qwen2_vl import Qwen2VisionTransformerPretrainedModel
    hc = Qwen2VLVisionConfig(depth=3, embed_dim=64, hidden_size=40, mlp_ratio=2, num_heads=4, patch_size=14, spatial_merge_size=2,
                             temporal_patch_size=2)
    hc._attn_implementation = "eager"
    torch.manual_seed(1)
    hf = Qwen2VisionTransformerPretrainedModel(hc).eval().float()
    cfg = QwenVisionConfig.from_hf(hc.to_dict())
    cfg.dtype = "float32"
    assert not cfg.gated_mlp and cfg.window_size == 0 and cfg.intermediate_size == 128 and cfg.out_hidden_size == 40
    enc = QwenVisionEncoder(cfg)
    assert enc.load_hf_state_dict(hf.state_dict(), prefix="") == []
    x = _patches(cfg, GRIDS, seed=2)
    with torch.no_grad():
        out = hf(x, grid_thw=torch.tensor(GRIDS))
    want = out.pooler_output if hasattr(out, "pooler_output") else out
    got = enc(x, GRIDS)
    assert (got - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item())


def test_rotary_rows_and_patchify():
    t = rotary_rows([(1, 4, 6)], 16, 2)
    assert t.shape == (24, 16)
    # block order: the first four patches are rows 0-1 × columns 0-1; row angles sit in pairs 0..3, column angles in 4..7
    inv0 = 1.0
    assert torch.allclose(t[1, 4], torch.cos(torch.tensor(1.0 * inv0))) and torch.allclose(t[2, 0], torch.cos(torch.tensor(1.0 * inv0)))
    assert torch.allclose(t[0, :8], torch.ones(8)) and torch.allclose(t[0, 8:], torch.zeros(8))
    cfg = QwenVisionConfig(depth=1, hidden_size=64, num_heads=1, intermediate_size=64, out_hidden_size=32, dtype="float32")
    img = torch.arange(3 * 56 * 84, dtype=torch.float32).reshape(1, 3, 56, 84)
    p, grid = patchify_frames(img, cfg)
    assert grid == (1, 4, 6) and p.shape == (24, 3 * 2 * 14 * 14)
    # patch 1 of the first block is row 0, column 1; channel 0, both temporal copies hold the same pixels
    first = p[1].reshape(3, 2, 14, 14)
    assert torch.equal(first[0, 0], img[0, 0, :14, 14:28]) and torch.equal(first[0, 1], first[0, 0])
    # patch 2 of the first block is row 1, column 0
    assert torch.equal(p[2].reshape(3, 2, 14, 14)[1, 0], img[0, 1, 14:28, :14])
    with pytest.raises(ValueError):
        patchify_frames(torch.zeros(1, 3, 50, 84), cfg)
    enc = QwenVisionEncoder(cfg).random_init(0)
    with pytest.raises(ValueError):
        enc(p[:-1], [grid])


def test_multimodal_runner_with_qwen_tower():
    """End to end: image bytes → smart resize → patches → tower → rows spliced into the prompt with grid-shaped 3-D positions."""
    import numpy as np
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime import native as rt
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.multimodal import MultimodalInputs, MultimodalRunner
    cfg = tiny_llama_config(num_hidden_layers=2, vocab_size=200, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                            dtype="float32")
    cfg.mrope_section = [2, 3, 3]
    llm = LLM(cfg, device="cpu", max_batch_size=1, max_input_len=256, max_kv_cache_capacity=320, page_size=16)
    vc = QwenVisionConfig(depth=2, hidden_size=64, num_heads=4, intermediate_size=64, out_hidden_size=64, window_size=56,
                          fullatt_block_indexes=[1], dtype="float32")
    tower = QwenVisionEncoder(vc).random_init(3)
    mm = MultimodalRunner(llm, vision=tower, image_token_id=7, min_pixels=28 * 28 * 4, max_pixels=28 * 28 * 40)
    rng = np.random.default_rng(0)
    wide = rng.integers(0, 255, (60, 170, 3), dtype=np.uint8)                 # → 56 × 168: grid 4 × 12 patches, 2 × 6 tokens
    tall = rng.integers(0, 255, (120, 50, 3), dtype=np.uint8)
    req = MultimodalInputs().text([3, 4]).image(wide).text([5]).image(tall).text([6, 8])
    ids, emb, pos3, delta = mm.build(req)
    g0, g1 = mm._grids
    assert g0 == (1, 2, 6) and g1[0] == 1 and g1[1] > g1[2]
    n0, n1 = g0[1] * g0[2], g1[1] * g1[2]
    assert ids.count(7) == n0 + n1 and emb.shape == (len(ids), 64)
    # positions of the first image: rows count 0..1, columns 0..5 from the text offset 2
    img0 = pos3[:, 2:2 + n0]
    assert img0[0].tolist() == [2] * n0 and img0[1].tolist() == [2 + r for r in range(2) for _ in range(6)]
    assert img0[2].tolist() == [2 + c for _ in range(2) for c in range(6)]
    assert delta == int(pos3.max()) + 1 - len(ids)
    out = mm.generate(req, max_tokens=4)
    assert len(out) == 4
    # PNG bytes go through the native decoder to the same rows
    PIL = pytest.importorskip("PIL.Image")
    import io
    buf = io.BytesIO()
    PIL.fromarray(wide).save(buf, "PNG")
    rows_png = mm.encode_images([buf.getvalue()])[0]
    rows_arr = mm.encode_images([wide])[0]
    assert torch.equal(rows_png, rows_arr)


def test_runner_from_a_vision_language_checkpoint(tmp_path):
    """A Qwen2.5-VL style directory (nested text_config, ``model.language_model.*`` and ``model.visual.*`` tensors) loads into the
    language model and the tower; the tower's rows equal the Hugging Face tower's."""
    import json
    import os
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel
    from tensorrt_edge_llm_b200.checkpoint import save_file
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.multimodal import MultimodalRunner
    vc = Qwen2_5_VLVisionConfig(depth=2, hidden_size=64, intermediate_size=64, num_heads=4, window_size=56, out_hidden_size=64,
                                fullatt_block_indexes=[1])
    vc._attn_implementation = "eager"
    torch.manual_seed(4)
    tower = Qwen2_5_VisionTransformerPretrainedModel(vc).eval().float()
    text = dict(model_type="qwen2_5_vl_text", vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True,
                rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, dtype="float32")
    g = torch.Generator().manual_seed(5)
    sd = {"model.visual." + k: v.contiguous() for k, v in tower.state_dict().items()}
    lm = "model.language_model."
    sd[lm + "embed_tokens.weight"] = torch.randn(160, 64, generator=g) * 0.05
    sd[lm + "norm.weight"] = torch.ones(64)
    for i in range(2):
        p = f"{lm}layers.{i}."
        for name, shape in (("self_attn.q_proj", (64, 64)), ("self_attn.k_proj", (32, 64)), ("self_attn.v_proj", (32, 64)), ("self_attn.o_proj", (64, 64)),
                            ("mlp.gate_proj", (128, 64)), ("mlp.up_proj", (128, 64)), ("mlp.down_proj", (64, 128))):
            sd[p + name + ".weight"] = torch.randn(*shape, generator=g) * 0.05
        for name, n in (("self_attn.q_proj", 64), ("self_attn.k_proj", 32), ("self_attn.v_proj", 32)):
            sd[p + name + ".bias"] = torch.randn(n, generator=g) * 0.05
        sd[p + "input_layernorm.weight"] = torch.ones(64)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(64)
    d = str(tmp_path)
    save_file(sd, os.path.join(d, "model.safetensors"))
    json.dump({"model_type": "qwen2_5_vl", "architectures": ["Qwen2_5_VLForConditionalGeneration"], "image_token_id": 150, "dtype": "float32",
               "text_config": text, "vision_config": vc.to_dict(), "tie_word_embeddings": True}, open(os.path.join(d, "config.json"), "w"))
    llm = LLM(d, device="cpu", max_batch_size=1, max_input_len=256, max_kv_cache_capacity=320, page_size=16)
    assert llm.cfg.mrope_section == [2, 3, 3] and llm.cfg.attention_bias
    mm = MultimodalRunner.from_pretrained(llm, d)
    assert mm is not None and mm.image_token_id == 150 and mm.vision.cfg.window_size == 56
    x = _patches(mm.vision.cfg, [(1, 4, 8)], seed=6)
    with torch.no_grad():
        want = tower(x, grid_thw=torch.tensor([[1, 4, 8]])).pooler_output
    assert (mm.vision(x, [(1, 4, 8)]) - want).abs().max() < 2e-4
    from tensorrt_edge_llm_b200.runtime.multimodal import MultimodalInputs
    import numpy as np
    img = np.random.default_rng(1).integers(0, 255, (56, 112, 3), dtype=np.uint8)
    out = mm.generate(MultimodalInputs().text([11, 12]).image(img).text([13]), max_tokens=3)
    assert len(out) == 3
    # a text-only checkpoint has no tower
    json.dump({"model_type": "llama", **text}, open(os.path.join(d, "config.json"), "w"))
    assert MultimodalRunner.from_pretrained(llm, d) is None


def test_qwen3_vl_tower_and_deepstack_match_hf():
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLVisionConfig
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLVisionModel
    hc = Qwen3VLVisionConfig(depth=4, hidden_size=64, intermediate_size=96, num_heads=4, patch_size=16, spatial_merge_size=2,
                             temporal_patch_size=2, out_hidden_size=48, num_position_embeddings=36, deepstack_visual_indexes=[0, 2])
    hc._attn_implementation = "eager"
    torch.manual_seed(7)
    hf = Qwen3VLVisionModel(hc).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or n.endswith("bias"):
                p.copy_(torch.randn_like(p) * 0.3 + (1.0 if n.endswith("weight") else 0.0))
    cfg = QwenVisionConfig.from_hf(hc.to_dict())
    cfg.dtype = "float32"
    assert cfg.mlp_act == "gelu_tanh" and cfg.patch_bias and cfg.num_position_embeddings == 36 and cfg.deepstack_visual_indexes == [0, 2]
    enc = QwenVisionEncoder(cfg)
    assert enc.load_hf_state_dict(hf.state_dict(), prefix="") == []
    x = _patches(cfg, GRIDS, seed=8)
    with torch.no_grad():
        out = hf(x, grid_thw=torch.tensor(GRIDS))
    rows, taps = enc(x, GRIDS, return_deepstack=True)
    scale = max(1.0, out.pooler_output.abs().max().item())
    assert (rows - out.pooler_output).abs().max() < 2e-4 * scale
    assert len(taps) == 2
    for got, want in zip(taps, out.deepstack_features):
        assert got.shape == want.shape and (got - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item())


def test_deepstack_features_reach_the_decoder():
    """A Qwen3-VL style tower feeds its deepstack levels to the language model's first layers through the runner."""
    import numpy as np
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.multimodal import MultimodalInputs, MultimodalRunner
    cfg = tiny_llama_config(num_hidden_layers=3, vocab_size=200, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                            dtype="float32")
    cfg.mrope_section = [2, 3, 3]
    llm = LLM(cfg, device="cpu", max_batch_size=1, max_input_len=256, max_kv_cache_capacity=320, page_size=16)
    vc = QwenVisionConfig(depth=3, hidden_size=64, num_heads=4, intermediate_size=64, out_hidden_size=64, window_size=0, fullatt_block_indexes=[],
                          gated_mlp=False, mlp_act="gelu_tanh", patch_bias=True, patch_size=16, num_position_embeddings=16,
                          deepstack_visual_indexes=[0, 1], dtype="float32")
    tower = QwenVisionEncoder(vc).random_init(5, std=0.2)
    mm = MultimodalRunner(llm, vision=tower, image_token_id=7, min_pixels=32 * 32 * 2, max_pixels=32 * 32 * 30)
    img = np.random.default_rng(2).integers(0, 255, (64, 96, 3), dtype=np.uint8)
    req = MultimodalInputs().text([3, 4]).image(img).text([5, 6])
    ids, emb, pos3, delta = mm.build(req)
    n_img = ids.count(7)
    assert n_img == 2 * 3 and sorted(mm.deepstack) == [0, 1]
    rows, feats = mm.deepstack[1]
    assert rows.tolist() == list(range(2, 2 + n_img)) and feats.shape == (n_img, 64)
    with_deep = mm.generate(req, max_tokens=1)
    # the same prompt without the deepstack levels gives different logits: run the prefill by hand
    runner = llm.runner
    llm.kv.free(0)
    a = runner.prefill_embeds([0], [emb], positions3=[pos3], rope_deltas=[delta], deepstack=mm.deepstack).clone()
    llm.kv.free(0)
    b = runner.prefill_embeds([0], [emb], positions3=[pos3], rope_deltas=[delta])
    llm.kv.free(0)
    assert (a - b).abs().max() > 1e-3 and int(a.argmax()) == with_deep[0]


def test_encoder_cache_serves_repeated_images_with_their_deepstack_levels():
    import numpy as np
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.multimodal import MultimodalRunner
    cfg = tiny_llama_config(num_hidden_layers=2, vocab_size=200, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                            dtype="float32")
    llm = LLM(cfg, device="cpu", max_batch_size=1, max_input_len=256, max_kv_cache_capacity=320, page_size=16)
    vc = QwenVisionConfig(depth=2, hidden_size=64, num_heads=4, intermediate_size=64, out_hidden_size=64, window_size=0, fullatt_block_indexes=[],
                          gated_mlp=False, mlp_act="gelu_tanh", patch_bias=True, patch_size=16, num_position_embeddings=16,
                          deepstack_visual_indexes=[0], dtype="float32")
    tower = QwenVisionEncoder(vc).random_init(5, std=0.2)
    calls = []
    fwd = tower.forward
    tower.forward = lambda *a, **k: (calls.append(len(a[1])), fwd(*a, **k))[1]
    mm = MultimodalRunner(llm, vision=tower, image_token_id=7, cache_bytes=1 << 20, min_pixels=32 * 32 * 2, max_pixels=32 * 32 * 30)
    rng = np.random.default_rng(4)
    a, b = (rng.integers(0, 255, (64, 96, 3), dtype=np.uint8) for _ in range(2))
    first = mm.encode_images([a, b])
    deep_first = [d.clone() for d in mm._deep]
    again = mm.encode_images([b, a, b])                                  # all cached: the tower does not run
    assert calls == [2] and mm.cache.hits == 3
    assert torch.equal(again[0], first[1]) and torch.equal(again[1], first[0]) and torch.equal(again[2], first[1])
    n = first[0].shape[0]
    assert torch.equal(mm._deep[0][n:2 * n], deep_first[0][:n])          # deepstack rows follow their image
    c = rng.integers(0, 255, (64, 96, 3), dtype=np.uint8)
    mixed = mm.encode_images([a, c])
    assert calls == [2, 1] and torch.equal(mixed[0], first[0])


def test_video_clip_takes_a_grid_with_a_time_axis():
    import numpy as np
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.multimodal import MultimodalInputs, MultimodalRunner
    cfg = tiny_llama_config(num_hidden_layers=2, vocab_size=200, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                            dtype="float32")
    cfg.mrope_section = [2, 3, 3]
    llm = LLM(cfg, device="cpu", max_batch_size=1, max_input_len=256, max_kv_cache_capacity=320, page_size=16)
    vc = QwenVisionConfig(depth=2, hidden_size=64, num_heads=4, intermediate_size=64, out_hidden_size=64, window_size=56,
                          fullatt_block_indexes=[1], dtype="float32")
    mm = MultimodalRunner(llm, vision=QwenVisionEncoder(vc).random_init(3), image_token_id=7, min_pixels=28 * 28 * 4, max_pixels=28 * 28 * 40)
    rng = np.random.default_rng(0)
    frames = [rng.integers(0, 255, (56, 84, 3), dtype=np.uint8) for _ in range(4)]      # four frames → two temporal steps of 2 × 3 tokens
    req = MultimodalInputs().text([3, 4]).video(frames).text([5])
    ids, emb, pos3, delta = mm.build(req)
    assert mm._grids == [(2, 2, 3)] and ids.count(7) == 12
    clip = pos3[:, 2:14]
    assert clip[0].tolist() == [2] * 6 + [3] * 6                      # the temporal component advances per grid step
    assert clip[1].tolist() == [2, 2, 2, 3, 3, 3] * 2 and clip[2].tolist() == [2, 3, 4] * 4
    assert len(mm.generate(req, max_tokens=3)) == 3
    still = MultimodalInputs().text([3, 4]).image(frames[0]).text([5])
    assert mm.build(still)[0].count(7) == 6
