"""Vision encoder on CPU against a plain PyTorch statement of the same blocks, and image-row merging into a prompt."""
import torch
import torch.nn.functional as F

from tensorrt_edge_llm_b200.models.vit import VisionConfig, VisionEncoder, merge_image_embeddings


def _plain(enc: VisionEncoder, patches):
    c = enc.cfg
    n, t, _ = patches.shape
    x = F.linear(patches.reshape(n * t, -1), enc.patch_embed.weight, enc.patch_embed.bias) + enc.pos_embed[:t].repeat(n, 1)
    for b in enc.blocks:
        y = F.layer_norm(x, (c.hidden_size,), b.norm1.weight, b.norm1.bias, c.layer_norm_eps)
        q, k, v = F.linear(y, b.qkv.weight, b.qkv.bias).view(n, t, 3, c.num_attention_heads, c.head_dim).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v).permute(0, 2, 1, 3).reshape(n * t, c.hidden_size)
        x = x + F.linear(a, b.proj.weight, b.proj.bias)
        y = F.layer_norm(x, (c.hidden_size,), b.norm2.weight, b.norm2.bias, c.layer_norm_eps)
        x = x + F.linear(F.gelu(F.linear(y, b.fc1.weight, b.fc1.bias)), b.fc2.weight, b.fc2.bias)
    x = F.layer_norm(x, (c.hidden_size,), enc.norm.weight, enc.norm.bias, c.layer_norm_eps)
    m, g = c.spatial_merge, int(t ** 0.5)
    x = x.view(n, g // m, m, g // m, m, c.hidden_size).permute(0, 1, 3, 2, 4, 5).reshape(n * (g // m) ** 2, m * m * c.hidden_size)
    return F.linear(F.gelu(F.linear(x, enc.merger_fc1.weight, enc.merger_fc1.bias)), enc.merger_fc2.weight, enc.merger_fc2.bias)


def test_encoder_matches_plain_pytorch_and_merges_into_prompt():
    cfg = VisionConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256, patch_size=4, image_size=32,
                       out_hidden_size=96, dtype="float32")
    enc = VisionEncoder(cfg).random_init(0, std=0.1)
    g = torch.Generator().manual_seed(1)
    images = torch.randn(2, 3, 32, 32, generator=g)
    patches = VisionEncoder.patchify(images, 4)
    assert patches.shape == (2, 64, 48)
    assert torch.equal(patches[0, 9].view(3, 4, 4), images[0, :, 4:8, 4:8])        # patch 9 = row 1, column 1
    got, want = enc(patches), _plain(enc, patches)
    assert got.shape == (2 * 16, 96)
    assert (got - want).abs().max() < 2e-4
    ids = [1, 7, 7, 7, 5] + [7] * 29 + [2]
    text = torch.zeros(len(ids), 96)
    merged = merge_image_embeddings(ids, text, got, image_token_id=7)
    assert torch.equal(merged[1], got[0]) and torch.equal(merged[5], got[3]) and merged[0].abs().sum() == 0


def test_multimodal_prefill_through_runner():
    from tensorrt_edge_llm_b200 import AutoModel
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
    from tensorrt_edge_llm_b200.runtime.runner import ModelRunner
    model = AutoModel.from_config(tiny_llama_config(num_hidden_layers=2, dtype="float32"), random_init=0)
    h = model.cfg.hidden_size
    enc = VisionEncoder(VisionConfig(hidden_size=128, num_hidden_layers=1, num_attention_heads=2, intermediate_size=128, patch_size=4,
                                     image_size=16, out_hidden_size=h, dtype="float32")).random_init(1, std=0.1)
    img = enc(VisionEncoder.patchify(torch.randn(1, 3, 16, 16, generator=torch.Generator().manual_seed(2)), 4))      # 4 rows
    ids = [5, 9, 9, 9, 9, 11, 12]
    kv = KVCacheManager(model.cfg, num_pages=8, page_size=16, max_seats=2, max_pages_per_seq=4)
    r = ModelRunner(model, kv)
    merged = merge_image_embeddings(ids, r.embed_tokens(ids), img, image_token_id=9)
    with_image = r.prefill_embeds([0], [merged])
    text_only = r.prefill([1], [ids])
    assert with_image.shape == text_only.shape and not torch.allclose(with_image, text_only)
    # text-only embeddings through the embedding path reproduce the token path exactly
    kv.free(0)
    assert torch.allclose(r.prefill_embeds([0], [r.embed_tokens(ids)]), text_only, atol=1e-6)
    nxt = r.step([0], [[3]])                      # decoding continues from the multimodal prefix
    assert nxt.shape[0] == 1 and kv.lengths[0] == len(ids) + 1


def test_encoder_cache_and_data_parallel_shards():
    from tensorrt_edge_llm_b200.models.vit import EncoderCache, encode_data_parallel
    cfg = VisionConfig(hidden_size=128, num_hidden_layers=1, num_attention_heads=2, intermediate_size=256, patch_size=4, image_size=16,
                       out_hidden_size=32, dtype="float32")
    enc = VisionEncoder(cfg).random_init(0, std=0.1)
    patches = VisionEncoder.patchify(torch.randn(3, 3, 16, 16, generator=torch.Generator().manual_seed(2)), 4)
    want = enc(patches)
    calls = []

    def counted(x):
        calls.append(x.shape[0])
        return enc(x)
    cache = EncoderCache(budget_bytes=2 * 4 * 32 * 4 + 8)               # room for two images' rows
    assert torch.equal(cache.encode(counted, patches), want) and calls == [3]
    again = cache.encode(counted, patches[[2, 1, 0]])                   # image 0 was evicted by the budget, 1 and 2 are served
    assert torch.allclose(again, torch.cat([want[8:12], want[4:8], want[0:4]]), atol=1e-6) and calls == [3, 1] and cache.hits == 2
    assert cache.used <= cache.budget

    class FakeComm:                                                     # two ranks simulated in one process
        def __init__(self, rank, peers):
            self.world_size, self.rank, self.peers = 2, rank, peers

        def all_gather_rows(self, x):
            self.peers[self.rank] = x
            other = encode_rank(1 - self.rank) if self.peers[1 - self.rank] is None else self.peers[1 - self.rank]
            self.peers[1 - self.rank] = other
            return torch.cat([self.peers[0], self.peers[1]], 0)

    def encode_rank(r):
        per = 2
        idx = torch.arange(r * per, (r + 1) * per).clamp(max=2)
        return enc(patches[idx])
    out = encode_data_parallel(enc, patches, FakeComm(0, [None, None]))
    assert out.shape == want.shape and torch.allclose(out, want, atol=1e-6)


def test_dart_pruning_and_video_frame_sampling():
    from tensorrt_edge_llm_b200.models.vit import dart_prune, sample_video_frames
    g = torch.Generator().manual_seed(0)
    base = torch.randn(12, 32, generator=g)
    # 12 distinct rows, then 20 near-copies of row 3 (the row with the largest norm, hence a pivot)
    base[3] *= 4
    rows = torch.cat([base, base[3:4].repeat(20, 1) + 0.01 * torch.randn(20, 32, generator=g)])
    keep = dart_prune(rows, keep=14, num_pivots=2)
    kept = set(keep.tolist())
    assert keep.numel() == 14 and torch.equal(keep, keep.sort().values)
    family = {3} | set(range(12, 32))                           # 21 near-identical rows: only the pivots among them survive
    assert len(kept & family) == 3 and kept >= set(range(12)) - {3}
    assert torch.equal(dart_prune(rows, keep=100), torch.arange(32))
    idx = sample_video_frames(num_frames=300, video_fps=30.0, target_fps=2.0)
    assert len(idx) == 20 and idx[0] == 0 and idx[-1] == 299 and idx == sorted(idx)
    assert len(sample_video_frames(30, 30.0)) == 4              # short clip: the minimum
    assert len(sample_video_frames(100000, 25.0, max_frames=64)) == 64
    assert sample_video_frames(3, 30.0) == [0, 2]
