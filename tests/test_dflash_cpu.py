"""DFlash block-draft speculative decoding on tiny random models: losslessness, cache bookkeeping, acceptance."""
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import ModelConfig, tiny_llama_config
from tensorrt_edge_llm_b200.runtime.dflash import DFlashDecoder
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def _pair(block=6, shift=False, layers=2):
    tcfg = tiny_llama_config(num_hidden_layers=4, vocab_size=120, dtype="float32")
    target = AutoModel.from_config(tcfg, random_init=0)
    kv = KVCacheManager(tcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10)
    runner = ModelRunner(target, kv)
    dcfg = tiny_llama_config(num_hidden_layers=layers, vocab_size=120, dtype="float32")
    dcfg.draft_type, dcfg.dflash_block_size, dcfg.dflash_mask_token_id, dcfg.dflash_shift_label = "dflash", block, 119, shift
    dcfg.dflash_target_layer_ids = [0, 1, 3]
    draft = AutoModel.from_config(dcfg, random_init=1)
    assert type(draft).__name__ == "DFlashDraft"
    dkv = KVCacheManager(dcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10, num_layers=layers)
    return runner, draft, dkv, tcfg


def _greedy(tcfg, prompts, n):
    target = AutoModel.from_config(tcfg, random_init=0)
    kv = KVCacheManager(tcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10)
    r = ModelRunner(target, kv)
    first = r.prefill(list(range(len(prompts))), prompts).argmax(-1)
    rest = r.decode_greedy(list(range(len(prompts))), first, n - 1)
    return torch.cat([first[:, None], rest], 1).tolist()


def test_lossless_and_bookkeeping():
    for shift in (False, True):
        runner, draft, dkv, tcfg = _pair(block=6, shift=shift)
        dec = DFlashDecoder(runner, draft, dkv)
        prompts = [[5, 6, 7, 8, 9, 10, 11], [20, 21, 22]]
        out = dec.generate([0, 1], prompts, 24)
        assert out == _greedy(tcfg, prompts, 24)                       # exactly the target's greedy continuation
        # target cache: every emitted token but the last (the pending root); draft context rows: one per cached target token
        for s, p, o in zip([0, 1], prompts, out):
            assert runner.kv.lengths[s] == dkv.lengths[s]
            assert len(p) + len(o) - 1 <= runner.kv.lengths[s] + 6     # generation may overshoot the budget by less than a block
        assert dec.stats.rounds >= 4 and dec.stats.draft_forwards == dec.stats.rounds
        dec.release([0, 1])
        assert runner.kv.lengths[0] == 0 and dkv.lengths[0] == 0


def test_draft_that_knows_the_answer_is_accepted_whole():
    """Replace the draft's proposal with the target's own continuation: every round accepts block - 1 tokens."""
    runner, draft, dkv, tcfg = _pair(block=5)
    dec = DFlashDecoder(runner, draft, dkv)
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6]]
    want = _greedy(tcfg, prompts, 40)[0]
    pos = {"at": 1}

    def oracle(seats):
        d = torch.tensor([want[pos["at"]:pos["at"] + 4]])
        dec.stats.draft_forwards += 1
        return d
    dec._propose = oracle
    first = dec.prefill([0], prompts)
    assert first == [want[0]]
    got = list(first)
    for _ in range(4):
        new = dec.round([0])[0]
        assert len(new) == 5                                           # four drafts + the bonus token
        got += new
        pos["at"] += 5
    assert got == want[:21] and dec.stats.mean_accept_length == 5.0
    assert runner.kv.lengths[0] == len(prompts[0]) + 20 and dkv.lengths[0] == runner.kv.lengths[0]


def test_forced_accept_and_eos():
    runner, draft, dkv, tcfg = _pair(block=4)
    dec = DFlashDecoder(runner, draft, dkv)
    dec.prefill([0, 1], [[1, 2, 3], [4, 5, 6, 7]])
    new = dec.round([0, 1], forced_accept=[3, 1])
    assert [len(t) for t in new] == [4, 2]
    assert runner.kv.lengths[0] == 3 + 4 and runner.kv.lengths[1] == 4 + 2
    dec.release([0, 1])
    want = _greedy(tcfg, [[1, 2, 3]], 12)[0]
    eos = want[5]
    cut = dec.generate([0], [[1, 2, 3]], 12, eos_id=eos)[0]
    assert cut == want[:want.index(eos) + 1]


def test_context_rows_hold_projected_target_features():
    """The draft cache's keys are k_norm/RoPE(k_proj(norm(fc(taps)))) of the target rows — checked for layer 0, row 2."""
    from tensorrt_edge_llm_b200.ops import reference as ref
    runner, draft, dkv, tcfg = _pair(block=4)
    dec = DFlashDecoder(runner, draft, dkv)
    prompt = [9, 8, 7, 6, 5]
    dec.prefill([0], [prompt])
    meta = runner._meta([1], [5], logits_all=True)                     # recompute the taps on another seat
    x, taps = runner.model.hidden_states(torch.tensor(prompt, dtype=torch.int32), meta, runner.cache, capture_layers=[0, 1, 3])
    h = draft.project(torch.cat(taps, -1))
    a = draft.layers[0].self_attn
    qkv = a.qkv_proj(h)
    k = qkv[:, a.num_q_heads * a.head_dim:(a.num_q_heads + a.num_kv_heads) * a.head_dim].reshape(5, a.num_kv_heads, a.head_dim)
    if a.k_norm is not None:
        k = ref._head_rmsnorm(k, a.k_norm.weight, a.eps)
    k = ref.apply_rope(k, torch.arange(5), draft.cos_sin("cpu"))
    page = int(dkv.table_rows([0])[0, 0])
    assert (dkv.pool[0][page, 0, :, 2, :] - k[2]).abs().max() < 1e-5


def test_llm_with_a_dflash_draft_static_and_in_flight():
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    tcfg = tiny_llama_config(num_hidden_layers=4, vocab_size=120, dtype="float32")
    dcfg = tiny_llama_config(num_hidden_layers=2, vocab_size=120, dtype="float32")
    dcfg.draft_type, dcfg.dflash_block_size, dcfg.dflash_mask_token_id = "dflash", 5, 119
    prompts = [[5, 6, 7, 8], [20, 21, 22, 23, 24, 25]]
    plain = LLM(tcfg, device="cpu", max_batch_size=2, max_input_len=32, max_kv_cache_capacity=96, page_size=16)
    want = [o.token_ids for o in plain.generate(prompts, SamplingParams(max_tokens=18, ignore_eos=True))]
    llm = LLM(tcfg, device="cpu", max_batch_size=2, max_input_len=32, max_kv_cache_capacity=96, page_size=16, draft_model=dcfg)
    assert type(llm.spec_decoder).__name__ == "DFlashDecoder" and llm.spec_decoder.dkv.pool.shape[0] == 2
    outs = llm.generate(prompts, SamplingParams(max_tokens=18, ignore_eos=True))
    assert [o.token_ids for o in outs] == want and outs[0].spec_stats["verify_rounds"] >= 3
    # sampled requests are verified by rejection sampling along the chain
    samp = llm.generate(prompts[:1], SamplingParams(max_tokens=6, ignore_eos=True, temperature=0.8, top_k=20, seed=1))[0]
    assert len(samp.token_ids) == 6 and samp.spec_stats["verify_rounds"] >= 1
    ifb = LLM(tcfg, device="cpu", max_batch_size=2, max_input_len=32, max_kv_cache_capacity=96, page_size=16, draft_model=dcfg,
              enable_in_flight_batching=True)
    got = [o.token_ids for o in ifb.generate(prompts, SamplingParams(max_tokens=18, ignore_eos=True))]
    ifb.close()
    assert got == want


def test_domino_rollout_matches_a_literal_restatement_and_stays_lossless():
    """The correction head against a per-sequence loop with ``torch.nn.GRUCell`` (bias-free), and the decoder end to end."""
    tcfg = tiny_llama_config(num_hidden_layers=4, vocab_size=120, dtype="float32")
    target = AutoModel.from_config(tcfg, random_init=0)
    kv = KVCacheManager(tcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10)
    runner = ModelRunner(target, kv)
    dcfg = tiny_llama_config(num_hidden_layers=2, vocab_size=120, dtype="float32")
    dcfg.draft_type, dcfg.dflash_projector_type, dcfg.dflash_block_size, dcfg.dflash_mask_token_id = "dflash", "domino", 6, 119
    dcfg.domino_pool_size, dcfg.domino_proj_dim, dcfg.domino_gru_hidden_dim = 16, 8, 10
    draft = AutoModel.from_config(dcfg, random_init=1)
    assert type(draft).__name__ == "DominoDraft"
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for p in (draft.z_projection, draft.codebook, draft.gru_input_table, draft.gru_weight_hh, draft.proj_state_weight):
            p.copy_(torch.randn(p.shape, generator=g) * 0.5)
    dkv = KVCacheManager(dcfg, num_pages=32, page_size=16, max_seats=3, max_pages_per_seq=10, num_layers=2)
    dec = DFlashDecoder(runner, draft, dkv)
    prompts = [[5, 6, 7, 8, 9], [20, 21, 22]]
    dec.prefill([0, 1], prompts)
    got = dec._propose([0, 1])                                                   # [2, 5]
    # literal restatement from the block's hidden states
    from tensorrt_edge_llm_b200 import ops
    from tensorrt_edge_llm_b200.ops.meta import build_step_meta
    from tensorrt_edge_llm_b200.runtime.block_diffusion import full_mask
    ids = torch.full((2, 6), 119, dtype=torch.int32)
    ids[:, 0] = torch.tensor([dec.root[0], dec.root[1]], dtype=torch.int32)
    meta = build_step_meta([6, 6], [dkv.lengths[0], dkv.lengths[1]], dkv.table_rows([0, 1]), 16, slot_ids=[0, 1], logits_all=True,
                           tree_mask=full_mask(12, 6, "cpu"))
    x = draft.block_hidden(ops.embedding(ids.reshape(-1), draft.embed_tokens.weight), meta, dkv.pool).reshape(2, 6, -1)
    cell = torch.nn.GRUCell(1, 10, bias=False)
    with torch.no_grad():
        cell.weight_hh.copy_(draft.gru_weight_hh)
    def gru(tok, h):                                                             # x · W_ih is tabulated per token
        gi, gh = draft.gru_input_table[tok].float(), h @ cell.weight_hh.t()
        r = torch.sigmoid(gi[:10] + gh[:10]); z = torch.sigmoid(gi[10:20] + gh[10:20]); n = torch.tanh(gi[20:] + r * gh[20:])
        return (1 - z) * n + z * h
    for b in range(2):
        hid = x[b, 1:]
        logits = draft.head(hid)
        pool = torch.topk(logits.max(0).values, 16).indices
        want = [int(pool[logits[0, pool].argmax()])]
        h = gru(int(ids[b, 0]), torch.zeros(10))
        h = gru(want[0], h)
        for step in range(4):
            c = torch.nn.functional.silu(draft.z_projection.float() @ hid[step + 1] + draft.proj_state_weight.float() @ h)
            score = logits[step + 1, pool] + draft.codebook[pool].float() @ c
            want.append(int(pool[score.argmax()]))
            if step < 3:
                h = gru(want[-1], h)
        assert got[b].tolist() == want
    # the correction changes proposals but never the output: verification keeps it the target's greedy continuation
    dec.release([0, 1])
    assert dec.generate([0, 1], prompts, 20) == _greedy(tcfg, prompts, 20)


def test_sampled_requests_follow_the_target_distribution():
    """Second and third emitted token over many seeds against the exact marginals of the target model."""
    from tensorrt_edge_llm_b200.ops import reference as ref
    kw = dict(dtype="float32", vocab_size=12, hidden_size=64, intermediate_size=128, num_attention_heads=2, num_key_value_heads=1, head_dim=32)
    cfg = tiny_llama_config(num_hidden_layers=2, **kw)
    model = AutoModel.from_config(cfg, random_init=5)
    with torch.no_grad():
        model.lm_head.weight.mul_(8.0)                        # sharpen the distribution so that tokens differ in mass
    dcfg = tiny_llama_config(num_hidden_layers=1, **kw)
    dcfg.draft_type, dcfg.dflash_block_size, dcfg.dflash_mask_token_id = "dflash", 4, 11
    draft = AutoModel.from_config(dcfg, random_init=6)
    prompt = [3, 7, 1, 9, 5]
    temp = 0.9
    kv = KVCacheManager(cfg, num_pages=16, page_size=16, max_seats=1, max_pages_per_seq=4)
    r = ModelRunner(model, kv)
    p1 = ref.sampling_probs(r.prefill([0], [prompt]), temp)[0]
    exact2 = torch.zeros(12)
    for t1 in range(12):
        if p1[t1] < 1e-6:
            continue
        kv.free(0)
        r.prefill([0], [prompt])
        exact2 += p1[t1] * ref.sampling_probs(r.step([0], [[t1]]), temp)[0]
    dkv = KVCacheManager(dcfg, num_pages=16, page_size=16, max_seats=1, max_pages_per_seq=4, num_layers=1)
    dec = DFlashDecoder(r, draft, dkv)
    n = 700
    c1, c2 = torch.zeros(12), torch.zeros(12)
    multi = 0
    for seed in range(n):
        dec.release([0])
        rounds0 = dec.stats.rounds
        out = dec.generate([0], [prompt], 3, sampling={"temperature": temp, "top_k": 0, "top_p": 1.0, "seed": seed})[0]
        c1[out[0]] += 1
        c2[out[1]] += 1
        multi += int(dec.stats.rounds - rounds0 == 1)          # three tokens from one round: at least one draft was accepted
    tv1 = 0.5 * (c1 / n - p1).abs().sum()
    tv2 = 0.5 * (c2 / n - exact2).abs().sum()
    assert tv1 < 0.09 and tv2 < 0.09, (float(tv1), float(tv2))
    assert float(exact2.max()) < 0.9 and multi > 0
    # the same seed gives the same tokens; a cold temperature gives the greedy continuation
    dec.release([0])
    a = dec.generate([0], [prompt], 8, sampling={"temperature": temp, "top_k": 0, "top_p": 1.0, "seed": 3})
    dec.release([0])
    assert a == dec.generate([0], [prompt], 8, sampling={"temperature": temp, "top_k": 0, "top_p": 1.0, "seed": 3})
    dec.release([0])
    cold = dec.generate([0], [prompt], 8, sampling={"temperature": 0.01, "top_k": 0, "top_p": 1.0, "seed": 1})
    dec.release([0])
    assert cold == dec.generate([0], [prompt], 8)


def test_causal_block_variant_changes_proposals_not_outputs():
    """JetSpec-style drafts attend causally inside the block: other proposals, the same (target) output."""
    runner, draft, dkv, tcfg = _pair(block=6)
    dec = DFlashDecoder(runner, draft, dkv)
    prompts = [[5, 6, 7, 8, 9, 10, 11]]
    dec.prefill([0], prompts)
    full = dec._propose([0])
    draft.cfg.dflash_query_causal = True
    causal = dec._propose([0])
    assert full.shape == causal.shape == (1, 5) and not torch.equal(full, causal)
    dec.release([0])
    assert dec.generate([0], prompts, 16) == _greedy(tcfg, prompts, 16)
    from tensorrt_edge_llm_b200.config import ModelConfig
    hf = dict(model_type="qwen3", architectures=["JetSpecDraftModel"], vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
              num_attention_heads=4, num_key_value_heads=2, jetspec_config={"query_causal": True, "block_size": 8})
    c = ModelConfig.from_hf_dict(hf)
    assert c.draft_type == "dflash" and c.dflash_query_causal


def test_ddtree_assembly_is_the_best_prefix_set():
    """The assembled tree holds exactly the highest-scoring prefixes of the full candidate tree, prefix-closed, in
    non-increasing score order along every path; confidence and the survival floor steer and stop the growth."""
    import itertools

    from tensorrt_edge_llm_b200 import ops
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(2, 4, 30, generator=g) * 2.0
    ids, lp = ops.ddtree_candidates(logits, 3)
    assert ids.shape == (2, 4, 3) and torch.equal(ids[..., 0].long(), logits.argmax(-1)) and (lp[..., :-1] >= lp[..., 1:]).all()
    assert torch.allclose(lp, torch.log_softmax(logits, -1).gather(-1, ids.long()))
    n = 12
    tok, par, dep, sc, valid = ops.ddtree_assemble(ids, lp, torch.tensor([7, 9]), n)
    assert valid.tolist() == [n, n] and tok[:, 0].tolist() == [7, 9] and (sc[:, 0] == 0).all() and (par[:, 0] == 0).all()
    for i in range(2):
        # brute force: every prefix (slot choice per depth) with its score
        every = {}
        for d in range(1, 5):
            for slots in itertools.product(range(3), repeat=d):
                every[slots] = sum(float(lp[i, j, s]) for j, s in enumerate(slots))
        best = sorted(every.values(), reverse=True)[: n - 1]
        assert torch.allclose(sc[i, 1:].sort(descending=True).values, torch.tensor(best), atol=1e-5)
        paths = {0: ()}
        for j in range(1, n):
            p = int(par[i, j])
            assert p < j and int(dep[i, j]) == int(dep[i, p]) + 1 and float(sc[i, j]) <= float(sc[i, p]) + 1e-6     # prefix-closed
            slot = ids[i, int(dep[i, p])].tolist().index(int(tok[i, j]))
            paths[j] = paths[p] + (slot,)
            assert abs(every[paths[j]] - float(sc[i, j])) < 1e-5
        assert len(set(paths.values())) == n                                                           # no prefix twice
    # a depth the confidence head distrusts is reached later; below the survival floor it is not reached at all
    conf = torch.tensor([[1.0, 0.05, 1.0, 1.0], [1.0, 1.0, 1.0, 1.0]])
    _, _, dep_c, _, valid_c = ops.ddtree_assemble(ids, lp, torch.tensor([7, 9]), n, conf)
    assert dep_c[0, 1:4].tolist() == [1, 1, 1] and dep[0, 1:4].tolist() != [1, 1, 1]                  # every depth-1 candidate first
    assert torch.equal(dep_c[1], dep[1]) and valid_c.tolist() == [n, n]
    _, _, dep_s, sc_s, valid_s = ops.ddtree_assemble(ids, lp, torch.tensor([7, 9]), n, conf, 0.5)
    assert int(dep_s[0].max()) == 1 and valid_s.tolist() == [4, n] and torch.isinf(sc_s[0, 4:]).all()


def test_tree_verification_is_lossless_and_accepts_at_least_the_chain():
    prompts = [[5, 6, 7, 8, 9, 10, 11], [20, 21, 22]]
    runner, draft, dkv, tcfg = _pair(block=6)
    want = _greedy(tcfg, prompts, 24)
    chain = DFlashDecoder(runner, draft, dkv)
    assert chain.generate([0, 1], prompts, 24) == want
    chain_rounds = chain.stats.rounds
    chain.release([0, 1])
    for k, nodes in ((2, 10), (3, 16), (8, 64)):
        runner, draft, dkv, tcfg = _pair(block=6)
        dec = DFlashDecoder(runner, draft, dkv, tree_top_k=k, verify_tokens=nodes)
        assert dec.verify_tokens == nodes and dec.kv_headroom() == max(6, nodes)
        assert dec.generate([0, 1], prompts, 24) == want                # the target's greedy continuation, token for token
        # the tree's first chain is the chain decoder's proposal, so a round never accepts less
        assert dec.stats.rounds <= chain_rounds
        for s in (0, 1):
            assert runner.kv.lengths[s] == dkv.lengths[s]
        dec.release([0, 1])
    # the node budget is capped by what the candidate tree can hold, and drafts that propose tokens themselves are refused
    runner, draft, dkv, _ = _pair(block=3)
    assert DFlashDecoder(runner, draft, dkv, tree_top_k=2, verify_tokens=50).verify_tokens == 1 + 2 + 4
    import pytest
    with pytest.raises(ValueError, match="1..8"):
        DFlashDecoder(runner, draft, dkv, tree_top_k=9)


def test_llm_front_end_switches_block_drafts_to_tree_verification():
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    from tensorrt_edge_llm_b200.runtime.speculative import SpecConfig
    tcfg = tiny_llama_config(num_hidden_layers=4, vocab_size=120, dtype="float32")
    dcfg = tiny_llama_config(num_hidden_layers=2, vocab_size=120, dtype="float32")
    dcfg.draft_type, dcfg.dflash_block_size, dcfg.dflash_mask_token_id = "dflash", 5, 119
    prompts = [[5, 6, 7, 8], [20, 21, 22, 23, 24, 25]]
    kw = dict(device="cpu", max_batch_size=2, max_input_len=32, max_kv_cache_capacity=96, page_size=16)
    plain = LLM(tcfg, **kw)
    want = [o.token_ids for o in plain.generate(prompts, SamplingParams(max_tokens=18, ignore_eos=True))]
    plain.close()
    llm = LLM(tcfg, draft_model=dcfg, speculative=SpecConfig(block_tree_top_k=3, verify_tokens=20), **kw)
    try:
        assert llm.spec_decoder.tree_top_k == 3 and llm.spec_decoder.verify_tokens == 20
        assert [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=18, ignore_eos=True))] == want
    finally:
        llm.close()
    chain = LLM(tcfg, draft_model=dcfg, speculative=SpecConfig(), **kw)          # the default stays one chain per round
    assert chain.spec_decoder.tree_top_k == 1 and chain.spec_decoder.verify_tokens == 0
    chain.close()
