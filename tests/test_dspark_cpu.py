"""DSpark on CPU: Markov chain, confidence scores and both length schedules against literal loops; checkpoint contract;
lossless decoding with shortened, ragged verification steps."""
import math

import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import ModelConfig, tiny_llama_config
from tensorrt_edge_llm_b200.models.dspark import DSparkDraft
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.dflash import DFlashDecoder
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

from test_dflash_cpu import _greedy


def test_markov_chain_against_loops():
    g = torch.Generator().manual_seed(0)
    b, p, v, r = 4, 5, 30, 6
    logits = torch.randn(b, p, v, generator=g)
    w1, w2 = torch.randn(v, r, generator=g), torch.randn(v, r, generator=g)
    first = torch.tensor([3, 7, 29, 0])
    logits[0, 1, 4] = logits[0, 1, 9] = 40.0
    w2[4] = w2[9] = 0.0                                           # a tie the correction cannot break: the lower id wins
    temps = torch.tensor([0.0, 0.9, 0.0, 1.4])
    uni = torch.rand(b, p, generator=g)
    got = ref.markov_chain_propose(logits, w1, w2, first, temps, uni)
    for i in range(b):
        prev = int(first[i])
        for s in range(p):
            row = logits[i, s] + w2 @ w1[prev]
            if temps[i] < 1e-3:
                tok = int(row.argmax())
            else:
                ps = torch.softmax(row / temps[i], 0)
                hit = (ps.cumsum(0) > uni[i, s]).nonzero()
                tok = int(hit[0]) if hit.numel() else v - 1
            assert int(got[i, s]) == tok
            prev = tok
    assert int(got[0, 1]) == 4
    assert torch.equal(ref.markov_chain_propose(logits, w1, w2, first)[[0, 2]], got[[0, 2]])


def test_confidence_and_schedules_against_loops():
    g = torch.Generator().manual_seed(1)
    b, p, h, r, v = 3, 6, 8, 4, 20
    hid, w1 = torch.randn(b, p, h, generator=g), torch.randn(v, r, generator=g)
    wt, bias = torch.randn(h + r, generator=g), torch.tensor([0.3])
    first, toks = torch.tensor([1, 2, 3]), torch.randint(0, v, (b, p), generator=g)
    for with_markov in (False, True):
        conf = ref.markov_confidence(hid, w1, wt if with_markov else wt[:h], bias, first, toks, with_markov)
        for i in range(b):
            for s in range(p):
                z = float(hid[i, s] @ wt[:h]) + 0.3
                if with_markov:
                    z += float(w1[int(first[i]) if s == 0 else int(toks[i, s - 1])] @ wt[h:])
                assert math.isclose(float(conf[i, s]), 1 / (1 + math.exp(-z)), rel_tol=1e-5)
    conf = torch.tensor([[0.9, 0.9, 0.5, 0.99, 0.99, 0.99], [0.2, 0.9, 0.9, 0.9, 0.9, 0.9], [0.99] * 6])
    assert ref.confidence_proposal_lengths(conf, "threshold", 0.5).tolist() == [2, 1, 6]          # 0.81 ≥ .5 > .405 ; .2 < .5 ; .94
    assert ref.confidence_proposal_lengths(conf, "threshold", 0.0).tolist() == [6, 6, 6]
    assert ref.confidence_proposal_lengths(conf, "threshold", 0.5, min_len=2, max_len=4).tolist() == [2, 2, 4]
    # sps: expected tokens per unit cost, literal
    for floor in (0.0, 0.3):
        got = ref.confidence_proposal_lengths(conf, "sps", floor).tolist()
        for i in range(3):
            surv, exp_t, best, sel = 1.0, 1.0, -1e9, 1
            for s in range(6):
                surv *= float(conf[i, s]); exp_t += surv
                score = exp_t / (0.5 + 1.0 + 0.45 * (s + 2) + 0.02 * (s + 1))
                if score > best:
                    best, sel = score, s + 1
                if floor > 0 and surv < floor:
                    break
            assert got[i] == sel
    with pytest.raises(ValueError):
        ref.confidence_proposal_lengths(conf, "other", 0.1)


def test_checkpoint_contract():
    base = {"model_type": "qwen3", "architectures": ["Qwen3DSparkModel"], "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
            "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256, "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
            "torch_dtype": "float32", "block_size": 7, "mask_token_id": 250, "target_layer_ids": [1, 2, 3], "markov_rank": 16,
            "markov_head_type": "vanilla", "enable_confidence_head": True, "confidence_head_with_markov": True}
    cfg = ModelConfig.from_hf_dict(base)
    assert cfg.draft_type == "dflash" and cfg.dflash_projector_type == "dspark" and cfg.dflash_shift_label
    assert (cfg.dflash_block_size, cfg.dflash_mask_token_id, cfg.dflash_target_layer_ids, cfg.dspark_markov_rank) == (7, 250, [1, 2, 3], 16)
    from tensorrt_edge_llm_b200.model import model_class_for
    assert model_class_for(cfg) is DSparkDraft
    m = AutoModel.from_config(cfg, random_init=0)
    assert tuple(m.markov_w1.shape) == (256, 16) and tuple(m.confidence_weight.shape) == (64 + 16,) and tuple(m.confidence_bias.shape) == (1,)
    nested = ModelConfig.from_hf_dict({**{k: v for k, v in base.items() if k not in ("markov_rank", "markov_head_type", "block_size")},
                                       "architectures": ["X"], "dspark_config": {"markov_rank": 8, "block_size": 5, "causal": True}})
    assert nested.dflash_projector_type == "dspark" and nested.dflash_block_size == 5 and nested.dflash_query_causal and nested.dspark_markov_rank == 8
    for change in (dict(markov_rank=0), dict(markov_head_type="gated"), dict(block_size=1)):
        with pytest.raises(ValueError):
            ModelConfig.from_hf_dict({**base, **change})
    assert DSparkDraft.checkpoint_key_remap("model.rotary_emb.inv_freq") is None and DSparkDraft.checkpoint_key_remap("markov_w1") == "markov_w1"


def _pair(block=6, confidence=True):
    tcfg = tiny_llama_config(num_hidden_layers=4, vocab_size=120, dtype="float32")
    runner = ModelRunner(AutoModel.from_config(tcfg, random_init=0), KVCacheManager(tcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10))
    dcfg = tiny_llama_config(num_hidden_layers=2, vocab_size=120, dtype="float32")
    dcfg.draft_type, dcfg.dflash_projector_type, dcfg.dflash_block_size, dcfg.dflash_mask_token_id, dcfg.dflash_shift_label = "dflash", "dspark", block, 119, True
    dcfg.dflash_target_layer_ids, dcfg.dspark_markov_rank = [0, 1, 3], 6
    dcfg.dspark_enable_confidence_head, dcfg.dspark_confidence_head_with_markov = confidence, True
    draft = AutoModel.from_config(dcfg, random_init=1)
    assert isinstance(draft, DSparkDraft)
    g = torch.Generator().manual_seed(4)
    with torch.no_grad():
        for name, p in draft.named_parameters():
            if name.startswith(("markov_", "confidence_")):
                p.copy_(torch.randn(p.shape, generator=g) * 0.7)
    dkv = KVCacheManager(dcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10, num_layers=2)
    return runner, draft, dkv, tcfg


def test_proposals_lengths_and_lossless_decoding():
    prompts = [[5, 6, 7, 8, 9, 10, 11], [20, 21, 22]]
    runner, draft, dkv, tcfg = _pair()
    dec = DFlashDecoder(runner, draft, dkv)
    dec.prefill([0, 1], prompts)
    got = dec._propose([0, 1])
    assert got.shape == (2, 5) and draft.last_confidence.shape == (2, 5)
    assert draft.last_proposal_lengths.tolist() == [5, 5]                          # threshold 0: the whole block
    dec.release([0, 1])
    want = _greedy(tcfg, prompts, 22)
    assert dec.generate([0, 1], prompts, 22) == want
    full_rows = dec.stats.rounds
    # a schedule that shortens proposals: still the target's continuation, through ragged verification steps
    for schedule in (("threshold", 0.45), ("sps", 0.3)):
        runner, draft, dkv, tcfg = _pair()
        draft.schedule, draft.max_proposal_len = schedule, 4
        dec = DFlashDecoder(runner, draft, dkv)
        seen = []
        orig = dec._target_step
        dec._target_step = lambda seats, rows, q_lens: (seen.append(list(q_lens)), orig(seats, rows, q_lens))[1]
        assert dec.generate([0, 1], prompts, 22) == want
        verify = [q for q in seen[1:]]
        assert all(2 <= v <= 5 for q in verify for v in q) and any(v < 5 for q in verify for v in q)
    assert full_rows >= 1
    # no confidence head: no schedule, full blocks
    runner, draft, dkv, tcfg = _pair(confidence=False)
    dec = DFlashDecoder(runner, draft, dkv)
    assert dec.generate([0, 1], prompts, 12) == _greedy(tcfg, prompts, 12) and draft.last_proposal_lengths is None
