"""Qwen-VL vision tower on the GPU path (padded 80 → 128 heads, per-row rotary tables, window and frame attention as
ragged bidirectional steps) against the CPU reference ops with the same weights."""
import pytest
import torch

from tensorrt_edge_llm_b200.models.qwen_vl_vision import QwenVisionConfig, QwenVisionEncoder

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("gated", [True, False])
def test_tower_gpu_matches_cpu(gated):
    cfg = QwenVisionConfig(depth=2, hidden_size=320, num_heads=4, intermediate_size=512, out_hidden_size=256,
                           window_size=56 if gated else 0, fullatt_block_indexes=[1] if gated else [], gated_mlp=gated, dtype="bfloat16")
    assert cfg.head_dim == 80 and cfg.padded_head_dim == 128
    grids = [(1, 8, 12), (2, 4, 4)]
    enc = QwenVisionEncoder(cfg).random_init(0, std=0.05)
    x = torch.randn(sum(t * h * w for t, h, w in grids), cfg.patch_dim, generator=torch.Generator().manual_seed(1)) * 0.5
    want = enc(x, grids).float()
    got = enc.cuda()(x.cuda(), grids).float().cpu()
    assert got.shape == want.shape == (x.shape[0] // 4, 256)
    assert (got - want).abs().max() < 0.05 * max(want.abs().max().item(), 1.0)


def test_qwen3_vl_tower_with_deepstack_gpu_matches_cpu():
    """Qwen3-VL variant: tanh-GELU MLP, biased patch embedding, interpolated position table and deepstack taps."""
    cfg = QwenVisionConfig(depth=3, hidden_size=256, num_heads=2, intermediate_size=512, out_hidden_size=256, window_size=0,
                           fullatt_block_indexes=[], gated_mlp=False, mlp_act="gelu_tanh", patch_bias=True, patch_size=16,
                           num_position_embeddings=36, deepstack_visual_indexes=[0, 2], dtype="bfloat16")
    grids = [(1, 8, 12), (2, 4, 4)]
    enc = QwenVisionEncoder(cfg).random_init(0, std=0.05)
    x = torch.randn(sum(t * h * w for t, h, w in grids), cfg.patch_dim, generator=torch.Generator().manual_seed(1)) * 0.5
    want, want_taps = enc(x, grids, return_deepstack=True)
    got, got_taps = enc.cuda()(x.cuda(), grids, return_deepstack=True)
    assert got.shape == want.shape == (x.shape[0] // 4, 256) and len(got_taps) == len(want_taps) == 2
    for g, w in [(got, want)] + list(zip(got_taps, want_taps)):
        assert (g.float().cpu() - w.float()).abs().max() < 0.06 * max(w.float().abs().max().item(), 1.0)
