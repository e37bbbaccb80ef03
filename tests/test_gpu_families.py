"""Model families whose GPU paths are otherwise only reached through CPU restatements: the InternVL vision tower, the
flow-matching action expert over a language model's cache, and the block drafts with correction heads (Domino, DFlash 2,
DSpark, LiLiCorr) under their decoder.  bf16 on the tcgen05 kernels against the same weights on the CPU reference ops."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

pytestmark = pytest.mark.gpu


def test_internvl_tower_gpu_matches_cpu():
    from tensorrt_edge_llm_b200.models.internvl_vision import InternVisionConfig, InternVisionEncoder
    cfg = InternVisionConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=2, intermediate_size=512, image_size=56, patch_size=14,
                             out_hidden_size=256, dtype="bfloat16")
    enc = InternVisionEncoder(cfg).random_init(0, std=0.05)
    px = torch.randn(3, 3, 56, 56, generator=torch.Generator().manual_seed(1))
    want = enc(px).float()
    got = enc.cuda()(px.cuda()).float().cpu()
    assert got.shape == want.shape
    assert (got - want).abs().max() < 0.06 * max(want.abs().max().item(), 1.0)


def test_action_expert_velocity_gpu_matches_cpu():
    from tensorrt_edge_llm_b200.models.action_expert import ActionConfig, ActionExpert
    from tensorrt_edge_llm_b200.runtime.block_diffusion import full_mask
    tcfg = tiny_llama_config(num_hidden_layers=3, vocab_size=512, dtype="bfloat16", hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                             head_dim=128, intermediate_size=1024)
    ac = ActionConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                      rope_theta=10000.0, n_diffusion_tokens=8, in_proj_hidden_size=64, in_proj_num_fourier_feats=8, in_proj_max_freq=2.0,
                      dtype="bfloat16")
    target = AutoModel.from_config(tcfg, random_init=0)
    expert = ActionExpert(ac).init_random(3, std=0.05)
    sd_t = {k: v.clone() for k, v in target.state_dict().items()}
    sd_e = {k: v.clone() for k, v in expert.state_dict().items()}
    prompt = [(5 * i + 1) % 500 for i in range(37)]
    x = torch.randn(1, 8, 2, generator=torch.Generator().manual_seed(1))

    def run(device):
        t = AutoModel.from_config(tcfg)
        t.load_state_dict(sd_t)
        e = ActionExpert(ac)
        e.load_state_dict(sd_e)
        t, e = t.to(device), e.to(device)
        r = ModelRunner(t, KVCacheManager(tcfg, num_pages=8, page_size=64, max_seats=2, max_pages_per_seq=4, device=device), device)
        r.use_cuda_graphs = False
        r.prefill([0], [prompt])
        meta = r._meta([0], [8], tree_mask=full_mask(8, 8, device))
        return e.velocity(x.to(device), torch.tensor([0.3], device=device), meta, r.cache).float().cpu()

    want, got = run(torch.device("cpu")), run(torch.device("cuda", 0))
    assert got.shape == want.shape == (1, 8, 2)
    assert (got - want).abs().max() < 0.08 * max(want.abs().max().item(), 1.0)


def _block_decoder(kind, dev):
    from tensorrt_edge_llm_b200.runtime.dflash import DFlashDecoder
    kw = dict(vocab_size=512, dtype="bfloat16", hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=1024)
    tcfg = tiny_llama_config(num_hidden_layers=3, **kw)
    dcfg = tiny_llama_config(num_hidden_layers=2, **kw)
    dcfg.draft_type, dcfg.dflash_block_size, dcfg.dflash_mask_token_id, dcfg.dflash_target_layer_ids = "dflash", 8, 511, [0, 1, 2]
    if kind == "domino":
        dcfg.dflash_projector_type, dcfg.domino_pool_size, dcfg.domino_proj_dim, dcfg.domino_gru_hidden_dim = "domino", 64, 32, 32
    elif kind == "dflash2":
        dcfg.dflash_version, dcfg.dflash2_selector_rank, dcfg.dflash2_selector_top_k = 2, 64, 8
    elif kind == "lilicorr":
        dcfg.dflash_version, dcfg.dflash_projector_type = 2, "lilicorr"
        dcfg.lilicorr_candidate_topk, dcfg.lilicorr_hidden_size, dcfg.lilicorr_num_layers, dcfg.lilicorr_num_heads = 4, 64, 2, 4
        dcfg.lilicorr_mlp_ratio, dcfg.lilicorr_factor_dim, dcfg.lilicorr_vector_eps, dcfg.lilicorr_logit_scale = 2.0, 32, 1e-6, 8.0
    elif kind == "dspark":
        dcfg.dflash_projector_type, dcfg.dflash_shift_label, dcfg.dspark_markov_rank = "dspark", True, 64
        dcfg.dspark_enable_confidence_head, dcfg.dspark_confidence_head_with_markov = True, True
    target = AutoModel.from_config(tcfg, device=dev, random_init=0)
    draft = AutoModel.from_config(dcfg, device=dev, random_init=1)
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for name, p in list(draft.named_parameters()) + list(draft.named_buffers()):
            if any(t in name for t in ("codebook", "base_kernel", "markov_", "confidence_", "z_projection", "gru_", "proj_state", "slot_bias",
                                       "embedding", "in_proj")) and p.dtype.is_floating_point:
                p.copy_((torch.randn(p.shape, generator=g) * 0.3).to(p.dtype))

    def runner():
        r = ModelRunner(target, KVCacheManager(tcfg, num_pages=12, page_size=64, max_seats=2, max_pages_per_seq=4, device=dev))
        r.use_cuda_graphs = False
        return r
    dkv = KVCacheManager(dcfg, num_pages=12, page_size=64, max_seats=2, max_pages_per_seq=4, device=dev, num_layers=2)
    return runner, DFlashDecoder(runner(), draft, dkv), draft


@pytest.mark.parametrize("kind", ["domino", "dflash2", "lilicorr", "dspark"])
def test_block_drafts_with_correction_heads_on_gpu(kind):
    """Whatever the draft proposes, verification keeps the output the target's greedy continuation (a long common prefix: bf16
    near-ties may flip a late token between an 8-row verification step and a 1-row decode step)."""
    dev = torch.device("cuda", 0)
    runner, dec, draft = _block_decoder(kind, dev)
    prompts = [[(7 * i + 3) % 500 for i in range(40)], [(11 * i + 5) % 500 for i in range(23)]]
    r = runner()
    first = r.prefill([0, 1], prompts).float().argmax(-1)
    want = torch.cat([first[:, None], r.decode_greedy([0, 1], first.to(torch.int32), 31).to(first.device)], 1).tolist()
    if kind == "dspark":
        draft.schedule, draft.max_proposal_len = ("threshold", 0.3), 6          # shortened, ragged verification steps
    got = dec.generate([0, 1], prompts, 32)
    for gseq, wseq in zip(got, want):
        same = next((i for i, (a, b) in enumerate(zip(gseq, wseq)) if a != b), len(wseq))
        assert same >= 10, (kind, same, gseq, wseq)
    assert dec.stats.rounds >= 4
    torch.cuda.synchronize()
