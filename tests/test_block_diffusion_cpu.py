"""Block-diffusion decoding: the sampler's canvas policy against a literal per-position restatement, and the decoder on a
tiny random model (bidirectional canvas pass = hand-built dense attention mask; committed KV = a plain causal pass)."""
import json
import os

import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import DiffusionConfig, ModelConfig
from tensorrt_edge_llm_b200.runtime import block_diffusion as bd
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def _budget_loop(e, valid, bound):
    keep = [False] * len(e)
    order = sorted(range(valid), key=lambda i: (e[i], i))
    total = 0.0
    for i in order:
        if total > bound:                     # entropy kept so far (without the candidate) must stay within the bound
            break
        keep[i] = True
        total += max(e[i], 0.0)
    return keep


def test_entropy_budget_matches_loop():
    g = torch.Generator().manual_seed(0)
    for bound in (0.0, 0.1, 0.5, 3.0):
        e = torch.rand(5, 12, generator=g) * 0.4
        valid = torch.tensor([12, 7, 1, 12, 3])
        got = bd.entropy_budget(e, valid, bound)
        for b in range(5):
            assert got[b].tolist() == _budget_loop(e[b].tolist(), int(valid[b]), bound)
        assert got[:, 0].any() and got.sum(1).min() >= 1            # the most certain position is always kept
    assert not bd.entropy_budget(torch.rand(2, 4), torch.tensor([4, 4]), -1.0).any()


def test_sample_rows_entropy_and_distribution():
    logits = torch.tensor([[0.0, 0.0, 0.0, 0.0], [10.0, 0.0, 0.0, 0.0]])
    s, a, e = bd.sample_rows(logits, 1.0, torch.Generator().manual_seed(1))
    assert a.tolist()[1] == 0 and abs(float(e[0]) - 1.386294) < 1e-4 and float(e[1]) < 0.01
    # Gumbel-max draws follow softmax(logits / T)
    row = torch.tensor([[2.0, 1.0, 0.0]]).repeat(20000, 1)
    s, _, _ = bd.sample_rows(row, 0.5, torch.Generator().manual_seed(2))
    freq = torch.bincount(s, minlength=3).float() / 20000
    want = torch.softmax(torch.tensor([4.0, 2.0, 0.0]), 0)
    assert (freq - want).abs().max() < 0.015


def test_update_canvas_stability_and_convergence():
    cfg = DiffusionConfig(canvas_length=4, stability_window=2, entropy_threshold=0.05, entropy_bound=0.1)
    g = torch.Generator().manual_seed(3)
    st = bd.init_canvas(2, 4, 50, g, "cpu")
    valid = torch.tensor([4, 4])
    arg = torch.tensor([[1, 2, 3, 4], [5, 6, 7, 8]])
    low = torch.full((2, 4), 0.001)
    high = torch.tensor([[0.001] * 4, [0.001, 2.0, 2.0, 0.001]])
    for k in range(3):
        bd.update_canvas(st, arg.clone(), arg.clone(), high.clone(), valid, cfg, 50, False, g)
        assert st.stable[0].tolist() == [k + 1] * 4
        if k < 2:
            assert st.prefix.tolist() == [0, 0]
    # row 0: stable for 3 > window passes and mean entropy under the threshold → converged, canvas = arg-max
    assert st.prefix.tolist() == [4, 0] and st.canvas[0].tolist() == [1, 2, 3, 4]
    # row 1 is stable but too uncertain; the budget counts all kept positions but the largest, so the two certain
    # positions and the first uncertain one are kept and the last one is re-noised
    assert st.accepted[1].tolist() == [True, True, False, True] and st.canvas[1, 0] == 5 and st.canvas[1, 3] == 8
    # a converged row is frozen: later passes with other arg-maxes leave it alone; the forced pass fills the rest
    other = torch.tensor([[9, 9, 9, 9], [11, 12, 13, 14]])
    bd.update_canvas(st, other, other, low, valid, cfg, 50, True, g)
    assert st.argmax.tolist() == [[1, 2, 3, 4], [11, 12, 13, 14]] and st.prefix.tolist() == [4, 4]
    assert abs(bd.denoise_temperature(cfg, 0, 4) - 0.8) < 1e-6 and abs(bd.denoise_temperature(cfg, 3, 4) - 0.5) < 1e-6


def test_full_mask_bits():
    m = bd.full_mask(3, 40, "cpu")
    assert m.shape == (3, 2) and int(m[0, 0]) == -1 and int(m[0, 1]) == 255
    assert int(bd.full_mask(1, 32, "cpu")[0, 0]) == -1 and int(bd.full_mask(1, 31, "cpu")[0, 0]) == 2 ** 31 - 1


def _tiny(canvas=8, steps=6, **kw):
    hf = dict(model_type="diffusion_gemma", vocab_size=96, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=8, sliding_window=0, layer_types=["full_attention"] * 2,
              max_position_embeddings=256, dtype="float32", eos_token_id=95,
              diffusion=dict(canvas_length=canvas, max_denoising_steps=steps, **kw))
    cfg = ModelConfig.from_hf_dict(hf)
    model = AutoModel.from_config(cfg, random_init=0)
    kv = KVCacheManager(cfg, num_pages=32, page_size=16, max_seats=4, max_pages_per_seq=8)
    return cfg, model, ModelRunner(model, kv)


def test_config_and_registry():
    cfg, model, _ = _tiny(canvas=8, steps=6, entropy_bound=0.2)
    assert type(model).__name__ == "DiffusionGemmaLM" and cfg.diffusion.canvas_length == 8 and cfg.diffusion.entropy_bound == 0.2
    back = ModelConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert back.diffusion == cfg.diffusion
    gen = {"max_denoising_steps": 12, "t_max": 0.9, "sampler_config": {"_cls_name": "EntropyBoundSampler", "entropy_bound": 0.3}}
    d = DiffusionConfig.from_hf({"canvas_length": 64}, gen)
    assert (d.canvas_length, d.max_denoising_steps, d.t_max, d.entropy_bound, d.sampler_type) == (64, 12, 0.9, 0.3, "entropy_bound")


def test_canvas_pass_is_bidirectional_and_commit_is_causal():
    cfg, model, r = _tiny()
    prompt = [3, 9, 27, 81, 5, 15, 45]
    r.prefill([0], [prompt])
    canvas = torch.tensor([11, 22, 33, 44, 55, 66, 77, 88])
    x = model.canvas_inputs(canvas, None)
    meta = r._meta([0], [8], logits_all=True, tree_mask=bd.full_mask(8, 8, "cpu"))
    got = model(None, meta, r.cache, inputs_embeds=x)
    assert r.kv.lengths[0] == len(prompt)                               # nothing committed by a denoise pass
    # oracle: permuting the canvas rows together with their positions leaves each row's logits unchanged only when
    # every canvas row sees every other one — a causal pass would change them
    perm = torch.tensor([7, 6, 5, 4, 3, 2, 1, 0])
    pos = [len(prompt) + int(p) for p in perm]
    meta2 = r._meta([0], [8], logits_all=True, tree_mask=bd.full_mask(8, 8, "cpu"), positions=pos)
    got2 = model(None, meta2, r.cache, inputs_embeds=x[perm])
    assert (got2 - got[perm]).abs().max() < 1e-4
    causal = model(None, r._meta([0], [8], logits_all=True), r.cache, inputs_embeds=x)
    assert (causal[0] - got[0]).abs().max() > 1e-3                      # first row: a causal pass sees no later canvas row


def test_self_conditioning_math():
    cfg, model, _ = _tiny()
    sc = model.self_conditioning
    tok = torch.randn(5, 32)
    soft = torch.randn(5, 32)
    with torch.no_grad():
        sc.pre_norm.weight.copy_(torch.rand(32) + 0.5)
    rms = lambda v, w: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w
    xn = rms(soft, sc.pre_norm.weight)
    gu = xn @ sc.gate_up_proj.weight.T
    inter = gu.shape[-1] // 2
    want = rms(tok + (torch.nn.functional.gelu(gu[:, :inter], approximate="tanh") * gu[:, inter:]) @ sc.down_proj.weight.T,
               torch.ones(32))
    assert (sc(tok, soft, model.comm) - want).abs().max() < 1e-5
    logits = torch.randn(3, 96)
    want_soft = torch.softmax(logits / 0.7, -1) @ (model.model.embed_tokens.weight * model.model.embed_scale)
    assert (model.soft_embeddings(logits, 0.7) - want_soft).abs().max() < 1e-5


def test_generate_commits_blocks_and_is_reproducible():
    cfg, model, r = _tiny(canvas=8, steps=5)
    dec = bd.BlockDiffusionDecoder(r)
    prompts = [[1, 2, 3, 4, 5], [7, 8, 9]]
    out = dec.generate([0, 1], prompts, max_tokens=20, eos_ids=[])
    assert [len(o) for o in out] == [20, 20]
    assert r.kv.lengths[0] == 25 and r.kv.lengths[1] == 23             # every generated token is committed
    assert dec.stats.blocks == 3 and dec.stats.commit_passes == 3 and all(1 <= p <= 5 for p in dec.stats.passes_per_block)
    # the committed cache equals a plain causal prefill of prompt + output: next-token logits agree
    nxt = r.step([0, 1], [[out[0][-1]], [out[1][-1]]], commit=False)   # re-feeding a token: only used as a probe of the cache
    cfg2, model2, r2 = _tiny(canvas=8, steps=5)
    ref = r2.prefill([0, 1], [prompts[0] + out[0] + [out[0][-1]], prompts[1] + out[1] + [out[1][-1]]])
    assert (nxt - ref).abs().max() < 1e-4
    again = bd.BlockDiffusionDecoder(r2).generate([2, 3], prompts, max_tokens=20, eos_ids=[])
    assert again == out                                                 # same seed, same tokens
    other = bd.BlockDiffusionDecoder(r2, seed=7).generate([2, 3], prompts, max_tokens=20, eos_ids=[])
    assert other != out


def test_generate_stops_at_end_token_and_budget():
    cfg, model, r = _tiny(canvas=8, steps=3)
    dec = bd.BlockDiffusionDecoder(r)
    base = dec.generate([0], [[4, 5, 6]], max_tokens=16, eos_ids=[])[0]
    stop = base[4]
    first = base.index(stop)
    cut = dec.generate([0], [[4, 5, 6]], max_tokens=16, eos_ids=[stop])[0]
    assert cut == base[:first + 1] and r.kv.lengths[0] == 3 + first + 1
    hook = dec.generate([0], [[4, 5, 6]], max_tokens=16, should_stop=lambda i, toks: len(toks) == 11)[0]
    assert hook == base[:11]
    short = dec.generate([0], [[4, 5, 6]], max_tokens=5)[0]
    assert short == base[:5]                                            # the canvas keeps its length; the commit is cut
    assert dec.effective_steps() == 3 and dec.effective_steps(2) == 2 and dec.effective_steps(99) == 3 and dec.kv_headroom() == 8


def test_llm_generate_routes_to_block_diffusion():
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams
    cfg, _, _ = _tiny(canvas=8, steps=4)
    llm = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=32, max_kv_cache_capacity=64, page_size=16)
    assert llm.kv.max_pages_per_seq == (64 + 8 + 15) // 16             # one canvas of headroom
    outs = llm.generate([[1, 2, 3], [4, 5, 6, 7]], SamplingParams(max_tokens=12, ignore_eos=True, seed=5))
    assert [len(o.token_ids) for o in outs] == [12, 12] and outs[0].spec_stats["blocks"] == 2
    assert 2 <= outs[0].spec_stats["denoise_passes"] <= 8
    again = llm.generate([[1, 2, 3], [4, 5, 6, 7]], SamplingParams(max_tokens=12, ignore_eos=True, seed=5, max_denoising_steps=2))
    assert again[0].spec_stats["denoise_passes"] <= 4
    with pytest.raises(ValueError):
        llm.generate([[1, 2]], SamplingParams(max_tokens=4, logprobs=2))
    with pytest.raises(ValueError):
        LLM(cfg, device="cpu", enable_in_flight_batching=True)
