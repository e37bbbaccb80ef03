"""EAGLE-4 drafts on CPU: the low-rank candidate head's ordering rules, the checkpoint switches and key names, and tree
decoding that stays lossless with every combination of the additions."""
import math

import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import ModelConfig, tiny_llama_config
from tensorrt_edge_llm_b200.model import model_class_for
from tensorrt_edge_llm_b200.models.eagle4 import Eagle4Draft
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.speculative import SpecConfig

from test_speculative_cpu import _decoder, _greedy, _target


def test_candidate_head_matches_dense_definition():
    g = torch.Generator().manual_seed(0)
    rows, hid, rank, vocab, kc = 5, 32, 8, 200, 12
    h = torch.randn(rows, hid, generator=g).half()
    down, up, head = (torch.randn(*s, generator=g).half() for s in ((rank, hid), (vocab, rank), (vocab, hid)))
    ids, lp = ref.low_rank_candidate_head(h, down, up, head, kc)
    assert ids.dtype == torch.int32 and ids.shape == (rows, kc) and lp.dtype == torch.float32
    scores = (h.float() @ down.float().t()).half().float() @ up.float().t()
    for r in range(rows):
        want_set = set(scores[r].topk(kc).indices.tolist())
        assert set(ids[r].tolist()) == want_set
        exact = head[ids[r].long()].float() @ h[r].float()
        assert torch.all(exact[:-1] >= exact[1:])                             # ordered by the exact logit
        assert torch.allclose(lp[r], exact - torch.logsumexp(exact, 0), atol=1e-5)
        assert math.isclose(float(lp[r].exp().sum()), 1.0, rel_tol=1e-5)


def test_candidate_rescore_ties_and_non_finite():
    hid = 8
    h = torch.ones(1, hid)
    head = torch.zeros(6, hid)
    head[1] = 0.5; head[4] = 0.5                       # equal logits: the smaller id first
    head[2] = 1.0
    head[3, 0] = float("inf")                          # non-finite logit: ranks last, log-probability -inf
    ids, lp = ref.candidate_rescore(h, head, torch.tensor([[4, 3, 2, 1, 0]]))
    assert ids.tolist() == [[2, 1, 4, 0, 3]]
    assert lp[0, 4] == float("-inf") and torch.isfinite(lp[0, :4]).all()
    assert math.isclose(float(lp[0, :4].exp().sum()), 1.0, rel_tol=1e-6)
    # low-rank ties and NaN scores: ties go to the smaller id, NaN is never picked while real scores remain
    down = torch.eye(hid)[:4]
    up = torch.zeros(6, 4)
    up[5, 0] = float("nan")
    ids, _ = ref.low_rank_candidate_head(h, down, up, head, 3)
    assert sorted(ids[0].tolist()) == [0, 1, 2]


def _hf_config(**extra):
    base = {"model_type": "llama", "architectures": ["Eagle4LlamaForCausalLM"], "hidden_size": 64, "intermediate_size": 128,
            "num_hidden_layers": 1, "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256, "target_hidden_size": 64,
            "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "torch_dtype": "float32"}
    base.update(extra)
    return base


def test_config_switches_and_rules():
    cfg = ModelConfig.from_hf_dict(_hf_config(fc_norm=True, norm_output=True, num_aux_hidden_states=3,
                                              efficient_lm_head_config={"type": "low_rank", "num_candidates": 16, "rank": 8}))
    assert cfg.draft_type == "eagle3" and cfg.is_eagle4_draft and model_class_for(cfg) is Eagle4Draft
    assert (cfg.eagle_fc_norm, cfg.eagle_norm_output, cfg.draft_candidate_rank, cfg.draft_candidate_count) == (True, True, 8, 16)
    plain = ModelConfig.from_hf_dict(_hf_config(draft_vocab_size=128))
    assert plain.draft_type == "eagle3" and not plain.is_eagle4_draft
    ids = ModelConfig.from_hf_dict(_hf_config(fc_norm=True, eagle_aux_hidden_state_layer_ids=[1, 5]))
    assert ids.eagle3_target_layer_ids == [1, 5] and ids.eagle3_num_target_layers == 2
    bad = [dict(norm_output=False, efficient_lm_head_config={"type": "low_rank", "num_candidates": 16, "rank": 8}),
           dict(norm_output=True, efficient_lm_head_config={"type": "dense", "num_candidates": 16, "rank": 8}),
           dict(norm_output=True, efficient_lm_head_config={"type": "low_rank", "num_candidates": 0, "rank": 8}),
           dict(norm_output=True, efficient_lm_head_config={"type": "low_rank", "num_candidates": 16, "rank": 12}),
           dict(norm_output=True, draft_vocab_size=128, efficient_lm_head_config={"type": "low_rank", "num_candidates": 16, "rank": 8}),
           dict(norm_output=True, final_logit_softcapping=30.0, efficient_lm_head_config={"type": "low_rank", "num_candidates": 16, "rank": 8}),
           dict(fc_norm=True, norm_before_residual=True),
           dict(fc_norm=True, num_aux_hidden_states=2, eagle_aux_hidden_state_layer_ids=[1, 2, 3])]
    for extra in bad:
        with pytest.raises(ValueError):
            ModelConfig.from_hf_dict(_hf_config(**extra))


def test_checkpoint_key_names():
    m = Eagle4Draft.checkpoint_key_remap
    assert m("embed_tokens.weight") is None and m("t2d") is None
    assert m("midlayer.self_attn.q_proj.weight") == "layers.0.self_attn.q_proj.weight"
    assert m("efficient_lm_head_down_proj.weight") == "candidate_head.down_proj.weight"
    assert m("efficient_lm_head.weight") == "candidate_head.up_proj.weight"
    assert m("fc_norm.1.weight") == "fc_norm.1.weight"


def _draft4(target_cfg, **kw):
    cfg = tiny_llama_config(num_hidden_layers=1, dtype="float32")
    cfg.draft_type, cfg.eagle3_target_hidden_size = "eagle3", target_cfg.hidden_size
    for k, v in kw.items():
        setattr(cfg, k, v)
    model = AutoModel.from_config(cfg, random_init=2)
    assert isinstance(model, Eagle4Draft)
    return model


@pytest.mark.parametrize("kw", [dict(eagle_fc_norm=True), dict(eagle_norm_output=True),
                                dict(eagle_fc_norm=True, eagle_norm_output=True, draft_candidate_rank=8, draft_candidate_count=6)])
def test_eagle4_tree_decoding_is_lossless(kw):
    model = _target()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, model.cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 13)]
    want = _greedy(model, prompts, 10)
    for spec in (SpecConfig(draft_steps=3, top_k=3, verify_tokens=10), SpecConfig(draft_steps=1, top_k=8, verify_tokens=5)):
        dec = _decoder(model, _draft4(model.cfg, **kw), spec)
        assert dec.generate([0, 1], prompts, 10) == want


def test_candidate_head_proposals_are_the_head_output():
    model = _target()
    draft = _draft4(model.cfg, eagle_norm_output=True, draft_candidate_rank=8, draft_candidate_count=6)
    lp = torch.stack((torch.tensor([[-0.1, -2.0, -3.0, -4.0, -5.0, -6.0]]), torch.tensor([[9., 3., 200., 1., 0., 7.]])), dim=-2)
    sc, tok = draft.pick(lp, 4)
    assert tok.tolist() == [[9, 3, 200, 1]] and sc.tolist() == [[pytest.approx(-0.1), -2.0, -3.0, -4.0]]
    sc2, tok2 = draft.pick(lp.reshape(1, 1, 12), 10)                          # flattened by a caller, k above the candidate count
    assert tok2.shape == (1, 1, 6) and tok2[0, 0].tolist() == [9, 3, 200, 1, 0, 7]
