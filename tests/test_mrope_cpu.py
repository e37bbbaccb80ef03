"""Multimodal RoPE: per-row tables vs the Hugging Face Qwen2-VL rotation, 3-D prompt positions, decode offsets."""
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def test_rows_match_hf_multimodal_rotation():
    from transformers.models.qwen2_vl.modeling_qwen2_vl import apply_multimodal_rotary_pos_emb
    d, sections, t = 32, [4, 6, 6], 11
    g = torch.Generator().manual_seed(0)
    pos3 = torch.randint(0, 50, (3, t), generator=g)
    q = torch.randn(1, 2, t, d, generator=g)
    k = torch.randn(1, 1, t, d, generator=g)
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
    freqs = pos3[:, None, :, None].float() * inv[None, None, None, :]          # [3, 1, T, D/2]
    emb = torch.cat([freqs, freqs], dim=-1)
    want_q, want_k = apply_multimodal_rotary_pos_emb(q, k, emb.cos(), emb.sin(), sections)
    rows = ref.mrope_rows(ref.rope_cos_sin(64, d, 10000.0), pos3, sections)
    assert rows.shape == (t, d)
    got_q = ref.apply_rope(q[0].permute(1, 0, 2), torch.arange(t), rows).permute(1, 0, 2)
    got_k = ref.apply_rope(k[0].permute(1, 0, 2), torch.arange(t), rows).permute(1, 0, 2)
    assert (got_q - want_q[0]).abs().max() < 1e-5 and (got_k - want_k[0]).abs().max() < 1e-5
    # equal components reduce to ordinary RoPE
    same = ref.mrope_rows(ref.rope_cos_sin(64, d, 10000.0), torch.arange(t).expand(3, t), sections)
    assert torch.equal(same, ref.rope_cos_sin(64, d, 10000.0)[:t])


def test_prompt_positions_with_an_image():
    IMG = 9
    # text text [image 1x4x6 patches → 2x3 rows after the 2x2 merge] text text
    ids = [1, 2] + [IMG] * 6 + [3, 4]
    pos3, delta = ref.mrope_positions(ids, IMG, [(1, 4, 6)], spatial_merge=2)
    assert pos3[0].tolist() == [0, 1, 2, 2, 2, 2, 2, 2, 5, 6]
    assert pos3[1].tolist() == [0, 1, 2, 2, 2, 3, 3, 3, 5, 6]
    assert pos3[2].tolist() == [0, 1, 2, 3, 4, 2, 3, 4, 5, 6]
    assert delta == 7 - 10                                     # the next text position is 7, three less than the row count
    txt, d0 = ref.mrope_positions([5, 6, 7], IMG, [])
    assert txt.tolist() == [[0, 1, 2]] * 3 and d0 == 0


def test_model_prefill_and_decode_with_mrope():
    """A decoder with ``mrope_section``: equal components reproduce the ordinary run; image positions change the logits,
    and decode rows continue from the shifted position."""
    cfg = tiny_llama_config(num_hidden_layers=2, vocab_size=300)
    cfg.mrope_section = [8, 12, 12]                            # head_dim 64 → 32 rotary pairs
    model = AutoModel.from_config(cfg, random_init=0)

    def runner():
        kv = KVCacheManager(cfg, num_pages=16, page_size=16, max_seats=2, max_pages_per_seq=8)
        return ModelRunner(model, kv)
    ids = [3, 4] + [9] * 6 + [5, 6, 7]
    r0 = runner()
    emb = r0.embed_tokens(ids)
    base = r0.prefill([0], [ids])
    r1 = runner()
    flat = torch.arange(len(ids)).expand(3, len(ids))
    assert torch.allclose(r1.prefill_embeds([0], [emb], positions3=[flat], rope_deltas=[0]), base, atol=1e-5)
    pos3, delta = ref.mrope_positions(ids, 9, [(1, 4, 6)])
    r2 = runner()
    img = r2.prefill_embeds([0], [emb], positions3=[pos3], rope_deltas=[delta])
    assert (img - base).abs().max() > 1e-3 and r2.rope_delta[0] == delta == -3
    # the decode row sits at cache slot 11 but rotates as position 8: same logits as a full pass with explicit positions
    nxt = int(img.argmax(-1))
    step = r2.step([0], [[nxt]])
    r3 = runner()
    full3 = torch.cat([pos3, torch.full((3, 1), len(ids) + delta, dtype=torch.int32)], dim=1)
    emb_all = torch.cat([emb, r3.embed_tokens([nxt])], 0)
    want = r3.prefill_embeds([0], [emb_all], positions3=[full3], rope_deltas=[delta])
    assert torch.allclose(step, want, atol=1e-4)
    # a later sequence on the same seat starts clean
    r2.kv.free(0)
    assert torch.allclose(r2.prefill([0], [ids]), base, atol=1e-5) and 0 not in r2.rope_delta


def test_rope_scalings_match_hf():
    """dynamic-NTK and longrope tables against the Hugging Face initialisers."""
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    d, theta = 32, 10000.0

    def table(inv, att, n):
        ang = torch.arange(n, dtype=torch.float64)[:, None] * inv.double()[None, :]
        return torch.cat([ang.cos() * att, ang.sin() * att], -1).float()
    cfg = LlamaConfig(hidden_size=64, num_attention_heads=2, head_dim=d, max_position_embeddings=64, rope_theta=theta,
                      rope_scaling={"rope_type": "dynamic", "factor": 4.0})
    inv, att = ROPE_INIT_FUNCTIONS["dynamic"](cfg, "cpu", seq_len=256)
    got = ref.rope_cos_sin(256, d, theta, {"rope_type": "dynamic", "factor": 4.0, "original_max_position_embeddings": 64})
    assert (got - table(inv, att, 256)).abs().max() < 1e-4
    short, long_ = [1.0 + 0.05 * i for i in range(d // 2)], [2.0 + 0.3 * i for i in range(d // 2)]
    sc = {"rope_type": "longrope", "short_factor": short, "long_factor": long_, "factor": 4.0, "original_max_position_embeddings": 64}
    cfg = LlamaConfig(hidden_size=64, num_attention_heads=2, head_dim=d, max_position_embeddings=256, rope_theta=theta, rope_scaling=dict(sc))
    inv, att = ROPE_INIT_FUNCTIONS["longrope"](cfg, "cpu", seq_len=256)
    got = ref.rope_cos_sin(256, d, theta, sc)
    assert (got - table(inv, att, 256)).abs().max() < 1e-4
    inv_s, att_s = ROPE_INIT_FUNCTIONS["longrope"](cfg, "cpu", seq_len=32)
    got_s = ref.rope_cos_sin(64, d, theta, sc)
    assert (got_s - table(inv_s, att_s, 64)).abs().max() < 1e-4


def test_deepstack_features_join_the_early_layers():
    """Adding level features after layer k equals running the layers by hand with the addition in between."""
    cfg = tiny_llama_config(num_hidden_layers=3, vocab_size=300)
    model = AutoModel.from_config(cfg, random_init=0)
    kv = KVCacheManager(cfg, num_pages=8, page_size=16, max_seats=2, max_pages_per_seq=4)
    r = ModelRunner(model, kv)
    ids = [3, 4, 9, 9, 9, 5, 6]
    emb = r.embed_tokens(ids)
    base = r.prefill_embeds([0], [emb])
    g = torch.Generator().manual_seed(2)
    f0, f1 = torch.randn(3, cfg.hidden_size, generator=g) * 0.5, torch.randn(3, cfg.hidden_size, generator=g) * 0.5
    rows = [2, 3, 4]
    kv.free(0)
    got = r.prefill_embeds([0], [emb], deepstack={0: (rows, f0), 1: (rows, f1)})
    assert (got - base).abs().max() > 1e-3
    # by hand
    from tensorrt_edge_llm_b200 import ops
    kv.free(0)
    meta = r._meta([0], [len(ids)])
    cs = model.cos_sin("cpu")
    h, res = emb.clone(), None
    for i, layer in enumerate(model.model.layers):
        h, res = layer(h, res, meta, kv.pool[i], cs, model.comm)
        if i == 0:
            h[rows] += f0
        if i == 1:
            h[rows] += f1
    x, _ = ops.add_rmsnorm(h, res, model.model.norm.weight, model.model.norm.eps)
    want = model.logits_from_hidden(x, meta)
    assert torch.allclose(got, want, atol=1e-5)
