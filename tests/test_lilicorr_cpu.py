"""LiLiCorr on CPU: lattice bias and walk against literal loops, head output structure, contract, lossless block decoding."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import ModelConfig, tiny_llama_config
from tensorrt_edge_llm_b200.models.lilicorr import LiLiCorrDraft, lattice_attention_bias
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.dflash import DFlashDecoder
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

from test_dflash_cpu import _greedy


def test_lattice_bias_against_loops():
    g = torch.Generator().manual_seed(0)
    heads, slots, topk, block = 3, 4, 2, 5
    rel, same = torch.randn(heads, 2 * block - 1, generator=g), torch.randn(heads, generator=g)
    got = lattice_attention_bias(rel, same, slots, topk, block)
    assert got.shape == (heads, slots * topk, slots * topk) and got.dtype == torch.float32
    for h in range(heads):
        for q in range(slots * topk):
            for k in range(slots * topk):
                want = rel[h, q // topk - k // topk + block - 1] + (same[h] if q // topk == k // topk else 0.0)
                assert abs(float(got[h, q, k]) - float(want)) < 1e-6


def test_chain_walk_against_loops():
    g = torch.Generator().manual_seed(1)
    b, s, k = 5, 7, 4
    cand = torch.randint(0, 1000, (b, s, k), generator=g)
    tr = torch.randn(b, s, k, k, generator=g)
    tr[0, 2, :, 1] = tr[0, 2, :, 3] = 50.0                      # a tie: the lower index wins
    temps = torch.tensor([0.0, 0.7, 0.0, 1.2, 2.0])
    uni = torch.rand(b, s, generator=g)
    uni[3, 1] = 1.0                                              # clamped just below one
    tok, prob = ref.lattice_chain_walk(cand, tr, temps, uni)
    for i in range(b):
        prev = 0
        for j in range(s):
            row = tr[i, j, prev]
            if temps[i] < 1e-3:
                sel = int(row.argmax())
                p = torch.nn.functional.one_hot(torch.tensor(sel), k).float()
            else:
                p = torch.softmax(row / temps[i], 0)
                hit = (p.cumsum(0) > min(float(uni[i, j]), 0.99999994)).nonzero()
                sel = int(hit[0]) if hit.numel() else k - 1
            assert int(tok[i, j]) == int(cand[i, j, sel]) and torch.allclose(prob[i, j], p, atol=1e-6)
            prev = sel
    assert int(tok[0, 2]) == int(cand[0, 2, 1])
    tok_g, _ = ref.lattice_chain_walk(cand, tr)
    assert torch.equal(tok_g[0], tok[0]) and torch.equal(tok_g[2], tok[2])


def _hf(**dflash):
    return {"model_type": "qwen3", "architectures": ["LiLiCorrDraftModel"], "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
            "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256, "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
            "torch_dtype": "float32", "dflash_config": dflash}


_OK = dict(block_size=8, mask_token_id=255, is_causal=False, conv_kernel_size=2, conv_group_size=16, target_layer_ids=[1, 3], lilicorr_enabled=True,
           lilicorr_candidate_topk=4, lilicorr_hidden_size=32, lilicorr_num_layers=2, lilicorr_num_heads=4, lilicorr_mlp_ratio=2.0,
           lilicorr_factor_dim=16, lilicorr_vector_eps=1e-6, lilicorr_logit_scale=8.0)


def test_checkpoint_contract():
    cfg = ModelConfig.from_hf_dict(_hf(**_OK))
    assert cfg.draft_type == "dflash" and cfg.dflash_version == 2 and cfg.dflash_projector_type == "lilicorr"
    assert (cfg.lilicorr_candidate_topk, cfg.lilicorr_hidden_size, cfg.lilicorr_num_layers, cfg.lilicorr_logit_scale) == (4, 32, 2, 8.0)
    from tensorrt_edge_llm_b200.model import model_class_for
    assert model_class_for(cfg) is LiLiCorrDraft
    for change in (dict(lilicorr_enabled=False), dict(lilicorr_candidate_topk=3), dict(lilicorr_candidate_topk=32), dict(lilicorr_num_heads=0),
                   dict(target_layer_ids=[]), dict(is_causal=True)):
        with pytest.raises(ValueError):
            ModelConfig.from_hf_dict(_hf(**{**_OK, **change}))
    with pytest.raises(ValueError):
        ModelConfig.from_hf_dict(_hf(**{k: v for k, v in _OK.items() if k != "lilicorr_factor_dim"}))
    names = set(AutoModel.from_config(cfg, random_init=0).state_dict())
    for key in ("lilicorr.token_proj.weight", "lilicorr.feature_norm.bias", "lilicorr.layers.1.attn.in_proj_weight", "lilicorr.layers.0.mlp.up_proj.bias",
                "lilicorr.slot_embedding", "lilicorr.relative_slot_bias", "lilicorr.factor_input_proj.weight", "lilicorr.anchor_out_head.weight",
                "layers.0.attention_conv.base_kernel", "layers.1.mlp_conv.kernel_projection.weight"):
        assert key in names, key


def _pair(block=5):
    tcfg = tiny_llama_config(num_hidden_layers=4, vocab_size=120, dtype="float32")
    runner = ModelRunner(AutoModel.from_config(tcfg, random_init=0), KVCacheManager(tcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10))
    dcfg = tiny_llama_config(num_hidden_layers=2, vocab_size=120, dtype="float32")
    dcfg.draft_type, dcfg.dflash_version, dcfg.dflash_projector_type, dcfg.dflash_block_size, dcfg.dflash_mask_token_id = "dflash", 2, "lilicorr", block, 119
    dcfg.dflash_target_layer_ids, dcfg.dflash2_conv_group_size = [0, 1, 3], 8
    dcfg.lilicorr_candidate_topk, dcfg.lilicorr_hidden_size, dcfg.lilicorr_num_layers, dcfg.lilicorr_num_heads = 4, 32, 2, 4
    dcfg.lilicorr_mlp_ratio, dcfg.lilicorr_factor_dim, dcfg.lilicorr_vector_eps, dcfg.lilicorr_logit_scale = 2.0, 16, 1e-6, 8.0
    draft = AutoModel.from_config(dcfg, random_init=1)
    assert isinstance(draft, LiLiCorrDraft)
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for name, p in draft.named_parameters():
            if any(t in name for t in ("base_kernel", "embedding", "slot_bias", "in_proj", "feature_norm")):
                p.copy_(torch.randn(p.shape, generator=g) * 0.5)
    dkv = KVCacheManager(dcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10, num_layers=2)
    return runner, draft, dkv, tcfg


def test_head_scores_and_lossless_decoding():
    runner, draft, dkv, tcfg = _pair(block=5)
    dec = DFlashDecoder(runner, draft, dkv)
    prompts = [[5, 6, 7, 8, 9, 10, 11], [20, 21, 22]]
    dec.prefill([0, 1], prompts)
    assert set(draft._anchor) == {0, 1}
    hid = torch.randn(2, 4, tcfg.hidden_size, generator=torch.Generator().manual_seed(2))
    ids, scores = draft.lattice(hid, [0, 1])
    assert ids.shape == (2, 4, 4) and scores.shape == (2, 4, 4, 4) and scores.dtype == torch.float32
    assert torch.equal(scores[:, 0, 0], scores[:, 0, 3])                          # slot 0: the anchor scores for every `prev`
    assert float(scores.abs().max()) <= 8.0 + 1e-4                                # logit_scale times a cosine
    assert float((scores[:, 1:, 0] - scores[:, 1:, 1]).abs().max()) > 1e-3        # later slots depend on the previous candidate
    # a sequence without an anchor scores slot 0 with a zero anchor vector
    _, s2 = draft.lattice(hid[:1], [2])
    assert float(s2[:, 0].abs().max()) == 0.0
    got = dec._propose([0, 1])
    assert got.shape == (2, 4)
    dec.release([0, 1])
    assert dec.generate([0, 1], prompts, 20) == _greedy(tcfg, prompts, 20)
