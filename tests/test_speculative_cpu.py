"""EAGLE-3 tree speculative decoding on CPU: lossless against plain greedy decoding, with a random
draft (short acceptances) and with an oracle draft (every round accepts the whole chain)."""
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner
from tensorrt_edge_llm_b200.runtime.speculative import EagleDecoder, SpecConfig, default_tap_layers


def _target():
    cfg = tiny_llama_config(num_hidden_layers=4, dtype="float32")
    return AutoModel.from_config(cfg, random_init=1)


def _draft(target_cfg, draft_vocab=0):
    cfg = tiny_llama_config(num_hidden_layers=1, dtype="float32")
    cfg.draft_type = "eagle3"
    cfg.eagle3_target_hidden_size = target_cfg.hidden_size
    cfg.draft_vocab_size = draft_vocab
    return AutoModel.from_config(cfg, random_init=2)


def _greedy(model, prompts, n_new):
    kv = KVCacheManager(model.cfg, num_pages=64, page_size=16, max_seats=4, max_pages_per_seq=16)
    r = ModelRunner(model, kv)
    seats = list(range(len(prompts)))
    logits = r.prefill(seats, prompts)
    outs = [[int(t)] for t in logits.argmax(-1)]
    for _ in range(n_new - 1):
        logits = r.step(seats, [[o[-1]] for o in outs])
        for o, t in zip(outs, logits.argmax(-1)):
            o.append(int(t))
    return outs


def _decoder(model, draft, spec):
    kv = KVCacheManager(model.cfg, num_pages=64, page_size=16, max_seats=4, max_pages_per_seq=16)
    dkv = KVCacheManager(draft.cfg, num_pages=64, page_size=16, max_seats=4, max_pages_per_seq=16, num_layers=1)
    return EagleDecoder(ModelRunner(model, kv), draft, dkv, spec)


def test_tap_layers_and_mask_packing():
    assert default_tap_layers(36) == [2, 18, 33]
    assert len(default_tap_layers(2)) == 3
    parents = torch.tensor([[-1, 0, 0, 1, 3, 2]])
    anc = EagleDecoder._ancestors(parents)
    assert anc[0, 4].tolist() == [True, True, False, True, True, False]
    words = EagleDecoder._pack_mask(anc)
    assert words.shape == (6, 1) and int(words[4, 0]) == 0b011011
    big = EagleDecoder._pack_mask(torch.ones(1, 40, 40, dtype=torch.bool))
    assert big.shape == (40, 2) and int(big[0, 0]) == -1 and int(big[0, 1]) == 0xFF


def test_accept_and_commit_reference_ops():
    tree = torch.tensor([[9, 5, 6, 7, 8, 4]], dtype=torch.int32)
    par = torch.tensor([[-1, 0, 0, 1, 3, 2]], dtype=torch.int32)
    tgt = torch.tensor([[5, 7, 0, 8, 1, 0]], dtype=torch.int32)          # root→1 (5) →3 (7) →4 (8) → bonus 1
    path, plen, bonus = ref.spec_accept_greedy(tgt, tree, par, max_path=5)
    assert plen.tolist() == [4] and path[0, :4].tolist() == [0, 1, 3, 4] and bonus.tolist() == [1]
    path, plen, bonus = ref.spec_accept_greedy(tgt, tree, par, max_path=5, force_len=2)
    assert plen.tolist() == [2] and path[0, :2].tolist() == [0, 1]
    pool = torch.arange(2 * 4 * 2 * 1 * 4 * 2, dtype=torch.float32).view(2, 4, 2, 1, 4, 2).clone()
    before = pool.clone()
    table = torch.tensor([[2, 0, 3, -1]], dtype=torch.int32)
    path = torch.tensor([[0, 2, 5, 0]], dtype=torch.int32)
    ref.kv_commit_path(pool, table, torch.tensor([3]), path, torch.tensor([3]))
    # slot 3+2=5 → 3+1=4 ; slot 3+5=8 → 3+2=5   (page size 4: slot s lives in page table[s // 4], row s % 4)
    assert torch.equal(pool[:, 0, :, :, 0], before[:, 0, :, :, 1])        # slot 4 ← old slot 5 (page 0 rows 0 ← 1)
    assert torch.equal(pool[:, 0, :, :, 1], before[:, 3, :, :, 0])        # slot 5 ← old slot 8 (page 3 row 0)
    assert torch.equal(pool[:, 2], before[:, 2])                           # committed prefix untouched


def test_random_draft_is_lossless():
    model = _target()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, model.cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 17)]
    want = _greedy(model, prompts, 12)
    for spec in (SpecConfig(draft_steps=3, top_k=3, verify_tokens=10), SpecConfig(draft_steps=1, top_k=4, verify_tokens=5)):
        dec = _decoder(model, _draft(model.cfg), spec)
        got = dec.generate([0, 1], prompts, 12)
        assert got == want
        assert dec.stats.mean_accept_length >= 1.0


def test_reduced_draft_vocab_maps_through_d2t():
    model = _target()
    draft = _draft(model.cfg, draft_vocab=64)
    draft.d2t.copy_(torch.arange(64, dtype=torch.int32) * 3)
    prompts = [[1, 2, 3, 4, 5]]
    dec = _decoder(model, draft, SpecConfig(draft_steps=2, top_k=2, verify_tokens=6))
    assert dec.generate([0], prompts, 8) == _greedy(model, prompts, 8)


class _OracleDraft(torch.nn.Module):
    """Predicts the true greedy continuation: the row at position p proposes token p + 2 of the stream."""

    def __init__(self, draft, streams):
        super().__init__()
        self.cfg, self.d2t, self.streams = draft.cfg, draft.d2t, streams

    def forward(self, embeds, feature, meta, kv_pool):
        v = self.d2t.numel()
        rows = meta.logits_idx.long()
        lp = torch.full((rows.numel(), v), -30.0) - torch.arange(v) * 1e-3
        for j, r in enumerate(rows.tolist()):
            s, p = int(meta.seq_ids[r]), int(meta.positions[r])
            seq = self.streams[int(meta.slot_ids[s])]
            if p + 2 < len(seq):
                lp[j, seq[p + 2]] = 0.0
        return lp, torch.zeros(embeds.shape[0], self.cfg.hidden_size)


def test_oracle_draft_accepts_whole_chain():
    model = _target()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, model.cfg.vocab_size, (n,), generator=g).tolist() for n in (6, 11)]
    want = _greedy(model, prompts, 21)
    streams = {i: prompts[i] + want[i] for i in range(2)}
    spec = SpecConfig(draft_steps=4, top_k=2, verify_tokens=12)
    dec = _decoder(model, _OracleDraft(_draft(model.cfg), streams), spec)
    got = dec.generate([0, 1], prompts, 21)
    assert got == want
    assert dec.stats.mean_accept_length > 4.5            # depth 4 + bonus = 5 tokens per round until the stream ends


def test_forced_acceptance_length():
    model = _target()
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6]]
    dec = _decoder(model, _draft(model.cfg), SpecConfig(draft_steps=4, top_k=2, verify_tokens=12, force_accept_len=3))
    dec.prefill([0], prompts)
    for _ in range(4):
        assert len(dec.round([0])[0]) == 3
    assert dec.r.kv.lengths[0] == len(prompts[0]) + 12 and dec.dkv.lengths[0] == dec.r.kv.lengths[0]


def test_mtp_head_is_lossless_and_shares_lm_head():
    model = _target()
    cfg = tiny_llama_config(num_hidden_layers=1, dtype="float32")
    cfg.draft_type = "mtp"
    head = AutoModel.from_config(cfg, random_init=4)
    assert type(head).__name__ == "MtpDraft"
    head.share_lm_head(model)
    assert head.lm_head is model.lm_head
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, model.cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 13)]
    want = _greedy(model, prompts, 10)
    dec = _decoder(model, head, SpecConfig(draft_steps=3, top_k=1, verify_tokens=4))       # a chain of three drafts
    assert dec.taps == [model.cfg.num_hidden_layers - 1]
    assert dec.generate([0, 1], prompts, 10) == want
    assert MtpDraftRemap("mtp.fc.weight") == "fc.weight" and MtpDraftRemap("mtp.layers.0.mlp.up_proj.weight") == "layers.0.mlp.up_proj.weight"


from tensorrt_edge_llm_b200.models.mtp import MtpDraft  # noqa: E402

MtpDraftRemap = MtpDraft.checkpoint_key_remap


def test_llm_generate_with_draft_model_is_lossless():
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams
    cfg = tiny_llama_config(num_hidden_layers=4, dtype="float32")
    dcfg = tiny_llama_config(num_hidden_layers=1, dtype="float32")
    dcfg.draft_type, dcfg.eagle3_target_hidden_size = "eagle3", cfg.hidden_size
    kw = dict(device="cpu", max_batch_size=2, max_input_len=64, max_kv_cache_capacity=128, page_size=16, random_init_seed=1)
    plain = LLM(cfg, **kw)
    spec = LLM(cfg, draft_model=dcfg, speculative=SpecConfig(draft_steps=3, top_k=2, verify_tokens=8), **kw)
    prompts = [[3, 1, 4, 1, 5], [9, 2, 6, 5, 3, 5, 8]]
    sp = SamplingParams(max_tokens=9, ignore_eos=True)
    a, b = plain.generate(prompts, sp), spec.generate(prompts, sp)
    assert [o.token_ids for o in a] == [o.token_ids for o in b]
    assert spec.spec_decoder.stats.rounds > 0 and spec.kv.lengths[0] == 0          # seats released afterwards
    # sampled requests fall back to ordinary decoding
    assert len(spec.generate(prompts, SamplingParams(max_tokens=4, temperature=0.8, ignore_eos=True))[0].token_ids) == 4


def test_hybrid_target_chain_verify_with_state_replay():
    """Mamba2 / DeltaNet target: chain verification, recurrent rows restored and replayed after a partial acceptance."""
    import pytest
    from tensorrt_edge_llm_b200.config import GdnConfig, MambaConfig, hybrid_nemotron_config
    cfg = hybrid_nemotron_config(num_hidden_layers=8, vocab_size=500, hidden_size=64, intermediate_size=128, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=16, dtype="float32", max_position_embeddings=512,
                                 mamba=MambaConfig(num_heads=4, head_dim=8, d_state=16, n_groups=2, conv_kernel=4),
                                 gdn=GdnConfig(num_k_heads=2, num_v_heads=4, head_k_dim=8, head_v_dim=8, conv_kernel=4))
    model = AutoModel.from_config(cfg, random_init=0)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (7, 13)]
    want = _greedy(model, prompts, 14)
    dcfg = tiny_llama_config(num_hidden_layers=1, dtype="float32", vocab_size=500, hidden_size=64, intermediate_size=128,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=16)
    dcfg.draft_type, dcfg.eagle3_target_hidden_size = "eagle3", 64
    draft = AutoModel.from_config(dcfg, random_init=2)
    with pytest.raises(ValueError):
        _decoder(model, draft, SpecConfig(draft_steps=3, top_k=2, verify_tokens=8))
    # random draft: almost every chain is cut short, so nearly every round replays
    dec = _decoder(model, draft, SpecConfig(draft_steps=3, top_k=1, verify_tokens=4))
    passes = []
    orig = model.hidden_states
    model.hidden_states = lambda *a, **k: (passes.append(1), orig(*a, **k))[1]
    assert dec.generate([0, 1], prompts, 14) == want and dec.stats.replays > 0
    # every replay ran from the recorded kernel inputs: one model pass per prefill / verification round, none for a commit
    assert dec.stats.recurrent_replays == dec.stats.replays
    with_record = len(passes)
    # the fallback (no record): the accepted prefix goes through the whole model again, same tokens, more passes
    dec = _decoder(model, draft, SpecConfig(draft_steps=3, top_k=1, verify_tokens=4))
    dec.use_recurrent_replay = False
    passes.clear()
    assert dec.generate([0, 1], prompts, 14) == want and dec.stats.recurrent_replays == 0 and len(passes) > with_record
    model.hidden_states = orig
    # oracle draft: whole chains are accepted, no replay until the streams end
    streams = {i: prompts[i] + want[i] for i in range(2)}
    dec = _decoder(model, _OracleDraft(draft, streams), SpecConfig(draft_steps=3, top_k=1, verify_tokens=4))
    assert dec.generate([0, 1], prompts, 14) == want
    assert dec.stats.mean_accept_length > 3.0
    # forced partial acceptance exercises restore + replay on every round and still matches
    dec = _decoder(model, _OracleDraft(draft, streams), SpecConfig(draft_steps=3, top_k=1, verify_tokens=4, force_accept_len=2))
    assert dec.generate([0, 1], prompts, 14) == want and dec.stats.replays >= 10
    # sampled requests: rejection sampling along the chain, the same state commit; with a sharply peaked target and a very low
    # temperature the draws are the arg-max, so the output is the greedy continuation again
    with torch.no_grad():
        model.lm_head.weight.mul_(400.0)
    peaked = _greedy(model, prompts, 12)
    dec = _decoder(model, draft, SpecConfig(draft_steps=3, top_k=1, verify_tokens=4))
    got = dec.generate([0, 1], prompts, 12, sampling={"temperature": 0.002, "top_k": 0, "top_p": 1.0, "seed": 3})
    assert got == peaked and dec.stats.recurrent_replays > 0


def test_sampled_acceptance_reference_follows_the_target_distribution():
    torch.manual_seed(0)
    v = 8
    p_root = torch.tensor([0.3, 0.05, 0.2, 0.1, 0.15, 0.05, 0.1, 0.05])
    probs = torch.zeros(1, 4, v)
    probs[0, 0] = p_root
    probs[0, 1:] = torch.softmax(torch.randn(3, v), -1)
    tree, par = torch.tensor([[7, 0, 2, 5]]), torch.tensor([[-1, 0, 0, 0]])
    n = 6000
    u = torch.rand(n, 1, 2, 4, generator=torch.Generator().manual_seed(1))
    cnt, accepted = torch.zeros(v), 0
    for k in range(n):
        path, plen, bonus = ref.spec_accept_sampling(probs, tree, par, 2, u[k])
        accepted += int(plen[0] > 1)
        cnt[int(tree[0, path[0, 1]]) if plen[0] > 1 else int(bonus[0])] += 1
    assert (cnt / n - p_root).abs().max() < 0.02
    assert abs(accepted / n - float(p_root[[0, 2, 5]].sum())) < 0.03           # a child is accepted exactly when its token is drawn
    pr = ref.sampling_probs(torch.tensor([[2.0, 1.0, 0.0, -1.0]]), 1.0, top_k=2)
    assert pr[0, 2:].sum() == 0 and abs(float(pr[0, 0]) - 0.7311) < 1e-3
    pr = ref.sampling_probs(torch.tensor([[2.0, 1.0, 0.0, -1.0]]), 1.0, top_p=0.7)
    assert pr[0, 2:].sum() == 0 and abs(float(pr.sum()) - 1) < 1e-6


def test_sampled_speculative_decoding_matches_plain_sampling_in_distribution():
    """Second emitted token over many seeds: its empirical distribution is the exact marginal of the target model."""
    cfg = tiny_llama_config(num_hidden_layers=2, dtype="float32", vocab_size=16, hidden_size=64, intermediate_size=128,
                            num_attention_heads=2, num_key_value_heads=1, head_dim=32)
    model = AutoModel.from_config(cfg, random_init=5)
    with torch.no_grad():
        model.lm_head.weight.mul_(8.0)                        # sharpen the distribution so that tokens differ in mass
    dcfg = tiny_llama_config(num_hidden_layers=1, dtype="float32", vocab_size=16, hidden_size=64, intermediate_size=128,
                             num_attention_heads=2, num_key_value_heads=1, head_dim=32)
    dcfg.draft_type, dcfg.eagle3_target_hidden_size = "eagle3", 64
    draft = AutoModel.from_config(dcfg, random_init=6)
    prompt = [3, 7, 1, 12, 5]
    temp = 0.9
    # exact marginal of the second token
    kv = KVCacheManager(cfg, num_pages=16, page_size=16, max_seats=1, max_pages_per_seq=4)
    r = ModelRunner(model, kv)
    p1 = ref.sampling_probs(r.prefill([0], [prompt]), temp)[0]
    exact = torch.zeros(16)
    for t1 in range(16):
        if p1[t1] < 1e-6:
            continue
        kv.free(0)
        r.prefill([0], [prompt])
        exact += p1[t1] * ref.sampling_probs(r.step([0], [[t1]]), temp)[0]
    dec = _decoder(model, draft, SpecConfig(draft_steps=2, top_k=3, verify_tokens=8))
    n = 700
    c1, c2 = torch.zeros(16), torch.zeros(16)
    for seed in range(n):
        dec.release([0])
        out = dec.generate([0], [prompt], 2, sampling={"temperature": temp, "top_k": 0, "top_p": 1.0, "seed": seed})[0]
        c1[out[0]] += 1
        c2[out[1]] += 1
    tv1 = 0.5 * (c1 / n - p1).abs().sum()
    tv2 = 0.5 * (c2 / n - exact).abs().sum()
    assert tv1 < 0.09 and tv2 < 0.09, (float(tv1), float(tv2))
    assert float(exact.max()) < 0.9                            # the check is not vacuous: mass is spread over several tokens


def test_speculative_decoding_under_in_flight_batching():
    """Requests arriving at different times share draft → verify rounds; every output equals plain greedy decoding."""
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    cfg = tiny_llama_config(num_hidden_layers=4, dtype="float32")
    dcfg = tiny_llama_config(num_hidden_layers=1, dtype="float32")
    dcfg.draft_type, dcfg.eagle3_target_hidden_size = "eagle3", cfg.hidden_size
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 40, 17, 5)]
    plain = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=64, max_kv_cache_capacity=128, page_size=16, random_init_seed=1)
    want = [o.token_ids for o in plain.generate(prompts, SamplingParams(max_tokens=11, ignore_eos=True))]
    plain.close()
    llm = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=64, max_kv_cache_capacity=128, page_size=16, random_init_seed=1,
              draft_model=dcfg, speculative=SpecConfig(draft_steps=3, top_k=2, verify_tokens=8), enable_in_flight_batching=True)
    outs = llm.generate(prompts, SamplingParams(max_tokens=11, ignore_eos=True))          # four requests over two seats
    assert [o.token_ids for o in outs] == want
    assert llm.spec_decoder.stats.rounds > 0 and llm.engine.metrics().completed == 4
    # streaming delivers several tokens per chunk and the same sequence
    streamed, sizes = [], []
    for toks, _ in llm.generate_stream(prompts[1], SamplingParams(max_tokens=11, ignore_eos=True)):
        streamed += toks
        sizes.append(len(toks))
    assert streamed == want[1]
    # opted-out and sampled requests run token by token beside the speculative ones
    rounds = llm.spec_decoder.stats.rounds
    hs = [llm.submit(prompts[0], SamplingParams(max_tokens=11, ignore_eos=True, disable_spec_decode=True)),
          llm.submit(prompts[2], SamplingParams(max_tokens=11, ignore_eos=True))]
    got = [h.get(60.0) for h in hs]
    assert got == [want[0], want[2]] and llm.spec_decoder.stats.rounds > rounds
    sampled = llm.generate([prompts[0]], SamplingParams(max_tokens=6, temperature=0.8, top_k=20, seed=4, ignore_eos=True))[0]
    assert len(sampled.token_ids) == 6
    llm.close()
