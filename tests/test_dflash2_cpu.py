"""DFlash 2 on CPU: the dynamic grouped convolution and the chain selector against literal loops, the checkpoint contract,
and block decoding that stays the target's greedy continuation."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import ModelConfig, tiny_llama_config
from tensorrt_edge_llm_b200.models.dflash2 import DFlash2Draft
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.dflash import DFlashDecoder
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

from test_dflash_cpu import _greedy


@pytest.mark.parametrize("taps,block,group", [(2, 5, 4), (3, 2, 8), (1, 4, 2), (4, 16, 16)])
def test_grouped_dynamic_conv_against_loops(taps, block, group):
    g = torch.Generator().manual_seed(taps * block)
    n, h = 3, 32
    x = torch.randn(n * block, h, generator=g)
    delta = torch.randn(n * block, taps, h // group, generator=g)
    base = torch.randn(taps, h, generator=g)
    res = torch.randn(n * block, h, generator=g)
    want = torch.zeros(n * block, h)
    for t in range(n * block):
        for c in range(h):
            for k in range(taps):
                if t % block >= k:
                    want[t, c] += (base[k, c] + delta[t, k, c // group]) * x[t - k, c]
    assert torch.allclose(ref.dflash2_grouped_dynamic_conv(x, delta, base, None, block, group), want, atol=1e-5)
    assert torch.allclose(ref.dflash2_grouped_dynamic_conv(x, delta, base, res, block, group), want + res, atol=1e-5)


def test_selector_walk_against_loops_greedy_and_sampled():
    g = torch.Generator().manual_seed(4)
    b, s, k, r, vocab = 4, 6, 5, 8, 40
    cand = torch.stack([torch.stack([torch.randperm(vocab, generator=g)[:k] for _ in range(s)]) for _ in range(b)])
    cand[1, 2, 3] = vocab + 7                                       # out of vocabulary: no bilinear term, still selectable
    unary = torch.randn(b, s, k, generator=g)
    unary[0, 1, 0] = unary[0, 1, 2] = 9.0                           # a tie on the unary part ...
    z = torch.randn(b, s, r, generator=g)
    pcb, qcb = torch.randn(vocab, r, generator=g) * 0.3, torch.randn(vocab, r, generator=g) * 0.3
    qcb[cand[0, 1, 0]] = qcb[cand[0, 1, 2]] = 0.0                   # ... that the bilinear term does not break: smaller id wins
    anchor = torch.tensor([3, 11, vocab + 1, 0])                    # one anchor outside the vocabulary
    temps = torch.tensor([0.0, 0.8, 0.0, 1.3])
    uni = torch.rand(b, s, generator=g)
    tok, prob = ref.dflash2_selector_walk(cand, unary, z, anchor, pcb, qcb, temps, uni)
    for i in range(b):
        prev = int(anchor[i])
        for j in range(s):
            q = pcb[prev] * z[i, j] if 0 <= prev < vocab else torch.zeros(r)
            sc = torch.stack([unary[i, j, c] + (qcb[cand[i, j, c]] @ q if int(cand[i, j, c]) < vocab else 0.0) for c in range(k)])
            if temps[i] < 1e-3:
                best = max(range(k), key=lambda c: (float(sc[c]), -int(cand[i, j, c])))
                want_p = torch.nn.functional.one_hot(torch.tensor(best), k).float()
            else:
                want_p = torch.softmax(sc / temps[i], 0)
                cum = want_p.cumsum(0)
                hit = (cum > uni[i, j]).nonzero()
                best = int(hit[0]) if hit.numel() else k - 1
            assert int(tok[i, j]) == int(cand[i, j, best])
            assert torch.allclose(prob[i, j], want_p, atol=1e-6)
            prev = int(cand[i, j, best])
    assert int(tok[0, 1]) == min(int(cand[0, 1, 0]), int(cand[0, 1, 2]))
    tok_g, prob_g = ref.dflash2_selector_walk(cand, unary, z, anchor, pcb, qcb)      # no temperatures: every row greedy
    assert torch.equal(tok_g[0], tok[0]) and torch.equal(tok_g[2], tok[2]) and bool((prob_g.sum(-1) == 1).all())


def _hf(**dflash):
    return {"model_type": "qwen3", "architectures": ["DFlash2DraftModel"], "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
            "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256, "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
            "torch_dtype": "float32", "dflash_config": dflash}


def test_checkpoint_contract():
    ok = dict(block_size=8, mask_token_id=255, is_causal=False, conv_kernel_size=2, conv_group_size=16, selector_rank=32, selector_top_k=16,
              target_layer_ids=[1, 3, 5, 7, 9], output_multiplier=0.5)
    cfg = ModelConfig.from_hf_dict(_hf(**ok))
    assert cfg.draft_type == "dflash" and cfg.dflash_version == 2 and cfg.dflash_block_size == 8 and cfg.dflash2_output_multiplier == 0.5
    assert (cfg.dflash2_conv_kernel_size, cfg.dflash2_conv_group_size, cfg.dflash2_selector_rank, cfg.dflash2_selector_top_k) == (2, 16, 32, 16)
    from tensorrt_edge_llm_b200.model import model_class_for
    assert model_class_for(cfg) is DFlash2Draft
    for change in (dict(is_causal=True), dict(block_size=17), dict(target_layer_ids=[1, 1, 2]), dict(output_multiplier=0.0),
                   dict(conv_group_size=3), dict(selector_top_k=64)):
        with pytest.raises(ValueError):
            ModelConfig.from_hf_dict(_hf(**{**ok, **change}))
    for missing in ("conv_kernel_size", "selector_rank", "is_causal"):
        with pytest.raises(ValueError):
            ModelConfig.from_hf_dict(_hf(**{k: v for k, v in ok.items() if k != missing}))
    m = DFlash2Draft.checkpoint_key_remap
    assert m("model.layers.0.attention_conv.base_kernel") == "layers.0.attention_conv.base_kernel"
    assert m("candidate_selector.predecessor_codebook") == "predecessor_codebook"
    assert m("candidate_selector.hidden_projection.weight") == "hidden_projection.weight"


def _pair(block=6):
    tcfg = tiny_llama_config(num_hidden_layers=4, vocab_size=120, dtype="float32")
    runner = ModelRunner(AutoModel.from_config(tcfg, random_init=0), KVCacheManager(tcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10))
    dcfg = tiny_llama_config(num_hidden_layers=2, vocab_size=120, dtype="float32")
    dcfg.draft_type, dcfg.dflash_version, dcfg.dflash_block_size, dcfg.dflash_mask_token_id = "dflash", 2, block, 119
    dcfg.dflash_target_layer_ids = [0, 1, 3]
    dcfg.dflash2_selector_rank, dcfg.dflash2_selector_top_k, dcfg.dflash2_conv_group_size = 8, 4, 8
    draft = AutoModel.from_config(dcfg, random_init=1)
    assert isinstance(draft, DFlash2Draft)
    g = torch.Generator().manual_seed(9)
    with torch.no_grad():
        for name, p in draft.named_parameters():
            if "codebook" in name or "base_kernel" in name:
                p.copy_(torch.randn(p.shape, generator=g) * 0.5)
    dkv = KVCacheManager(dcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10, num_layers=2)
    return runner, draft, dkv, tcfg


def test_block_decoding_is_lossless_and_uses_the_selector():
    runner, draft, dkv, tcfg = _pair(block=6)
    dec = DFlashDecoder(runner, draft, dkv)
    prompts = [[5, 6, 7, 8, 9, 10, 11], [20, 21, 22]]
    dec.prefill([0, 1], prompts)
    got = dec._propose([0, 1])                                                    # [2, 5]
    # restate the head from the block's hidden states: per-slot top-k, then the chain walk
    from tensorrt_edge_llm_b200 import ops
    from tensorrt_edge_llm_b200.ops.meta import build_step_meta
    from tensorrt_edge_llm_b200.runtime.block_diffusion import full_mask
    ids = torch.full((2, 6), 119, dtype=torch.int32)
    ids[:, 0] = torch.tensor([dec.root[0], dec.root[1]], dtype=torch.int32)
    meta = build_step_meta([6, 6], [dkv.lengths[0], dkv.lengths[1]], dkv.table_rows([0, 1]), 16, slot_ids=[0, 1], logits_all=True,
                           tree_mask=full_mask(12, 6, "cpu"))
    x = draft.block_hidden(ops.embedding(ids.reshape(-1), draft.embed_tokens.weight), meta, dkv.pool).reshape(2, 6, -1)[:, 1:]
    logits = draft.head(x.reshape(10, -1)).reshape(2, 5, -1)
    unary, cand = logits.topk(4, dim=-1)
    z = x @ draft.hidden_projection.weight.t()
    want, _ = ref.dflash2_selector_walk(cand, unary, z, ids[:, 0], draft.predecessor_codebook, draft.successor_codebook)
    assert torch.equal(got, want)
    assert not torch.equal(want, cand[..., 0])                                    # the bilinear term changed at least one slot
    dec.release([0, 1])
    assert dec.generate([0, 1], prompts, 24) == _greedy(tcfg, prompts, 24)
