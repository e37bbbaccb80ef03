"""Speculative-decoding kernels and the EAGLE-3 decoder on the GPU."""
import pytest
import torch

from tensorrt_edge_llm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cu():
    from tensorrt_edge_llm_b200.ops import cuda
    cuda.lib()
    return cuda


def _random_tree(g, b, n, vocab=50):
    par = torch.full((b, n), -1, dtype=torch.int32)
    for i in range(b):
        for c in range(1, n):
            par[i, c] = int(torch.randint(0, c, (1,), generator=g))
    return torch.randint(0, vocab, (b, n), generator=g, dtype=torch.int32), par


@pytest.mark.parametrize("b,n", [(1, 8), (5, 60), (16, 128)])
def test_spec_accept_greedy(cu, b, n):
    g = torch.Generator().manual_seed(n)
    tree, par = _random_tree(g, b, n, vocab=4)          # small vocabulary: long accepted paths
    tgt = torch.randint(0, 4, (b, n), generator=g, dtype=torch.int32)
    force = torch.randint(1, 6, (b,), generator=g, dtype=torch.int32)
    for fl in (0, 3, force):
        want = ref.spec_accept_greedy(tgt, tree, par, 7, fl)
        got = cu.spec_accept_greedy(tgt.cuda(), tree.cuda(), par.cuda(), 7, fl.cuda() if isinstance(fl, torch.Tensor) else fl)
        assert torch.equal(got[1].cpu(), want[1]) and torch.equal(got[2].cpu(), want[2])
        for i in range(b):
            m = int(want[1][i])
            assert torch.equal(got[0][i, :m].cpu(), want[0][i, :m])


@pytest.mark.parametrize("b,n", [(1, 10), (4, 60), (16, 128), (3, 33)])
def test_eagle_tree_meta_kernel(cu, b, n):
    """Ancestor mask, depth and positions of random trees (and of forests whose rows hang under an absent root)."""
    g = torch.Generator().manual_seed(b * 100 + n)
    _, par = _random_tree(g, b, n)
    forest = par.clone()
    forest[:, : min(5, n)] = -1                                          # several parentless rows, as in a draft step
    base = torch.randint(0, 3000, (b,), generator=g, dtype=torch.int32)
    for table, depth_base, off in ((par, 0, 0), (forest, 1, -1)):
        want = ref.eagle_tree_meta(table, base, depth_base, off)
        got = cu.eagle_tree_meta(table.cuda(), base.cuda(), depth_base, off)
        torch.cuda.synchronize()
        for w, gt in zip(want, got):
            assert torch.equal(gt.cpu(), w)


@pytest.mark.parametrize("b,k,steps,n", [(1, 10, 6, 60), (4, 4, 3, 12), (16, 10, 6, 60), (2, 8, 4, 128)])
def test_eagle_select_verify_kernel(cu, b, k, steps, n):
    """Pool → verification tree: same nodes, order, parents and depths as the sort-based formulation (ties included)."""
    g = torch.Generator().manual_seed(k * steps)
    pool = k + (steps - 1) * k * k
    # a pool shaped like the draft's: depth-1 candidates, then k*k children per later depth with non-increasing scores
    sc = [-(torch.rand(b, k, generator=g) * 2)]
    par = [torch.full((b, k), -1, dtype=torch.int32)]
    dep = [torch.ones(b, k, dtype=torch.int32)]
    front = torch.arange(k).expand(b, k)
    base = k
    for d in range(2, steps + 1):
        psc = torch.cat(sc, 1).gather(1, front)
        csc = psc[:, :, None] - (torch.rand(b, k, k, generator=g) * 2).round(decimals=1)     # rounded: equal scores occur
        sc.append(csc.reshape(b, -1))
        par.append(front[:, :, None].expand(b, k, k).reshape(b, -1).to(torch.int32))
        dep.append(torch.full((b, k * k), d, dtype=torch.int32))
        front = base + csc.reshape(b, -1).topk(k, dim=-1).indices
        base += k * k
    p_sc, p_par, p_dep = torch.cat(sc, 1), torch.cat(par, 1), torch.cat(dep, 1)
    assert p_sc.shape[1] == pool
    p_tok = torch.randint(0, 32000, (b, pool), generator=g, dtype=torch.int32)
    root = torch.randint(0, 32000, (b,), generator=g, dtype=torch.int32)
    keep = min(n - 1, pool)
    want = ref.eagle_select_verify(p_sc, p_tok, p_par, p_dep, root, keep)
    got = cu.eagle_select_verify(p_sc.cuda(), p_tok.cuda(), p_par.cuda(), p_dep.cuda(), root.cuda(), keep)
    torch.cuda.synchronize()
    for w, gt in zip(want, got):
        assert torch.equal(gt.cpu(), w)


@pytest.mark.parametrize("d,psz", [(128, 64), (64, 128)])
def test_kv_commit_path(cu, d, psz):
    g = torch.Generator().manual_seed(d)
    layers, pages, hkv, b = 3, 12, 2, 3
    pool = torch.randn(layers, pages, 2, hkv, psz, d, generator=g).bfloat16()
    table = torch.stack([torch.randperm(pages, generator=g)[:4] for _ in range(b)]).to(torch.int32)
    past = torch.tensor([psz - 3, 5, 2 * psz - 1], dtype=torch.int32)       # paths straddle page boundaries
    path = torch.tensor([[0, 2, 5, 9, 40], [0, 1, 2, 0, 0], [0, 7, 0, 0, 0]], dtype=torch.int32)
    plen = torch.tensor([5, 3, 1], dtype=torch.int32)
    want = pool.clone()
    ref.kv_commit_path(want, table, past, path, plen)
    got = pool.cuda()
    cu.kv_commit_path(got, table.cuda(), past.cuda(), path.cuda(), plen.cuda())
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), want)


def test_eagle_decoder_on_gpu(cu):
    from tensorrt_edge_llm_b200 import AutoModel
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
    from tensorrt_edge_llm_b200.runtime.runner import ModelRunner
    from tensorrt_edge_llm_b200.runtime.speculative import EagleDecoder, SpecConfig
    kw = dict(num_hidden_layers=4, hidden_size=512, intermediate_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
              vocab_size=2048, dtype="bfloat16")
    dev = torch.device("cuda", 0)
    model = AutoModel.from_config(tiny_llama_config(**kw), random_init=1, device=dev)
    dcfg = tiny_llama_config(**{**kw, "num_hidden_layers": 1})
    dcfg.draft_type, dcfg.eagle3_target_hidden_size = "eagle3", 512
    draft = AutoModel.from_config(dcfg, random_init=2, device=dev)

    def decoder(spec):
        kv = KVCacheManager(model.cfg, num_pages=32, page_size=64, max_seats=4, max_pages_per_seq=8, device=dev)
        dkv = KVCacheManager(dcfg, num_pages=32, page_size=64, max_seats=4, max_pages_per_seq=8, device=dev, num_layers=1)
        r = ModelRunner(model, kv)
        r.use_cuda_graphs = False
        return EagleDecoder(r, draft, dkv, spec)

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (50, 70)]
    # forced lengths: KV bookkeeping of target and draft stay in lock-step across page boundaries
    dec = decoder(SpecConfig(draft_steps=6, top_k=10, verify_tokens=60, force_accept_mean=3.5, force_seed=1))
    dec.prefill([0, 1], prompts)
    total = [0, 0]
    for _ in range(8):
        out = dec.round([0, 1])
        for i, e in enumerate(out):
            assert 1 <= len(e) <= 7
            total[i] += len(e)
    for i in range(2):
        assert dec.r.kv.lengths[i] == len(prompts[i]) + total[i] == dec.dkv.lengths[i]
    assert 2.0 < dec.stats.mean_accept_length < 5.0
    # real acceptance: every emitted token must be the target's arg-max given the emitted prefix (teacher forcing)
    dec = decoder(SpecConfig(draft_steps=3, top_k=4, verify_tokens=16))
    outs = dec.generate([2, 3], prompts, 24)
    kv = KVCacheManager(model.cfg, num_pages=32, page_size=64, max_seats=4, max_pages_per_seq=8, device=dev)
    r = ModelRunner(model, kv)
    r.use_cuda_graphs = False
    for i, (p, o) in enumerate(zip(prompts, outs)):
        logits = r.step([i], [p + o[:-1]], logits_all=True).float()
        top2 = logits[len(p) - 1:].topk(2, dim=-1)
        for j, t in enumerate(o):
            # bf16 kernels of different shapes may flip near-ties: accept the emitted token when it is
            # the arg-max or within a small margin of it
            assert t == int(top2.indices[j, 0]) or float(top2.values[j, 0] - logits[len(p) - 1 + j, t]) < 0.05


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,hid,vocab,kc", [(1, 64, 300, 5), (7, 1024, 4000, 64), (33, 4096, 20000, 200)])
def test_candidate_rescore_kernel(cu, dtype, rows, hid, vocab, kc):
    """Exact rescoring of an EAGLE-4 candidate set against the fp32 restatement: same ids in the same order (up to swaps of
    logits that differ by rounding only), log-probabilities within 2e-3, and a tie / non-finite case bit for bit."""
    g = torch.Generator().manual_seed(rows * kc)
    h = (torch.randn(rows, hid, generator=g) / hid ** 0.5).to(dtype)
    head = torch.randn(vocab, hid, generator=g).to(dtype)
    cand = torch.stack([torch.randperm(vocab, generator=g)[:kc] for _ in range(rows)]).to(torch.int32)
    want_ids, want_lp = ref.candidate_rescore(h, head, cand)
    got_ids, got_lp = cu.candidate_rescore(h.cuda(), head.cuda(), cand.cuda())
    got_ids, got_lp = got_ids.cpu(), got_lp.cpu()
    assert torch.all(got_lp[:, :-1] >= got_lp[:, 1:])
    for r in range(rows):
        assert sorted(got_ids[r].tolist()) == sorted(want_ids[r].tolist())
        by_id = {int(i): float(v) for i, v in zip(want_ids[r], want_lp[r])}
        assert max(abs(by_id[int(i)] - float(v)) for i, v in zip(got_ids[r], got_lp[r])) < 2e-3
    assert (got_ids == want_ids).float().mean() > 0.98
    # ties go to the smaller id; a non-finite logit ranks last with log-probability -inf
    h1 = torch.ones(1, 8, dtype=dtype)
    hd = torch.zeros(6, 8, dtype=dtype)
    hd[1] = 0.5; hd[4] = 0.5; hd[2] = 1.0; hd[3, 0] = float("inf")
    c1 = torch.tensor([[4, 3, 2, 1, 0]], dtype=torch.int32)
    ids, lp = cu.candidate_rescore(h1.cuda(), hd.cuda(), c1.cuda())
    wi, wl = ref.candidate_rescore(h1, hd, c1)
    assert ids.cpu().tolist() == wi.tolist() == [[2, 1, 4, 0, 3]]
    assert lp[0, 4].item() == float("-inf") and torch.allclose(lp.cpu()[0, :4], wl[0, :4], atol=1e-5)


def test_low_rank_candidate_head_on_gpu(cu):
    from tensorrt_edge_llm_b200 import ops
    g = torch.Generator().manual_seed(5)
    rows, hid, rank, vocab, kc = 9, 512, 64, 8000, 32
    h = (torch.randn(rows, hid, generator=g) / hid ** 0.5).half()
    down, up, head = (torch.randn(*s, generator=g).half() for s in ((rank, hid), (vocab, rank), (vocab, hid)))
    want_ids, want_lp = ref.low_rank_candidate_head(h, down, up, head, kc)
    ids, lp = ops.low_rank_candidate_head(h.cuda(), down.cuda(), up.cuda(), head.cuda(), kc)
    overlap = sum(len(set(a.tolist()) & set(b.tolist())) for a, b in zip(ids.cpu(), want_ids)) / (rows * kc)
    assert overlap > 0.97                                   # the low-rank scores differ by 16-bit rounding at the cut only
    same_top = ids.cpu()[:, 0] == want_ids[:, 0]
    assert same_top.float().mean() >= 0.75 and torch.allclose(lp.cpu()[same_top, 0], want_lp[same_top, 0], atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("taps,block,group,hid", [(2, 16, 16, 2048), (3, 5, 8, 256), (1, 2, 2, 64), (4, 8, 32, 1024)])
def test_dflash2_conv_kernel(cu, dtype, taps, block, group, hid):
    g = torch.Generator().manual_seed(taps * hid)
    n = 5
    x = torch.randn(n * block, hid, generator=g).to(dtype)
    delta = (torch.randn(n * block, taps, hid // group, generator=g) * 0.5).to(dtype)
    base = torch.randn(taps, hid, generator=g).to(dtype)
    res = torch.randn(n * block, hid, generator=g).to(dtype)
    for r in (None, res):
        want = ref.dflash2_grouped_dynamic_conv(x.float(), delta.float(), base.float(), None if r is None else r.float(), block, group)
        got = cu.dflash2_grouped_dynamic_conv(x.cuda(), delta.cuda(), base.cuda(), None if r is None else r.cuda(), block, group)
        assert got.dtype == dtype
        tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
        assert torch.allclose(got.float().cpu(), want, atol=tol * 4, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("b,s,k,r", [(1, 15, 16, 256), (6, 7, 5, 64), (3, 1, 32, 1024)])
def test_dflash2_selector_kernel(cu, dtype, b, s, k, r):
    g = torch.Generator().manual_seed(b * s * k)
    vocab = 500
    cand = torch.stack([torch.stack([torch.randperm(vocab, generator=g)[:k] for _ in range(s)]) for _ in range(b)])
    cand[0, 0, k - 1] = vocab + 3                                           # out-of-vocabulary candidate
    unary = torch.randn(b, s, k, generator=g) * 2
    z = torch.randn(b, s, r, generator=g).to(dtype)
    pcb, qcb = (torch.randn(vocab, r, generator=g) * (2.0 / r ** 0.5)).to(dtype), torch.randn(vocab, r, generator=g).to(dtype)
    anchor = torch.randint(0, vocab, (b,), generator=g)
    want_tok, want_p = ref.dflash2_selector_walk(cand, unary, z, anchor, pcb, qcb)
    tok, p = cu.dflash2_selector_walk(cand.cuda(), unary.cuda(), z.cuda(), anchor.cuda(), pcb.cuda(), qcb.cuda())
    assert torch.equal(tok.cpu(), want_tok) and torch.equal(p.cpu(), want_p)
    temps = torch.linspace(0.0, 1.5, b)
    uni = torch.rand(b, s, generator=g)
    want_tok, want_p = ref.dflash2_selector_walk(cand, unary, z, anchor, pcb, qcb, temps, uni)
    tok, p = cu.dflash2_selector_walk(cand.cuda(), unary.cuda(), z.cuda(), anchor.cuda(), pcb.cuda(), qcb.cuda(), temps.cuda(), uni.cuda())
    # a draw that lands within rounding of a bin edge may differ; everything downstream of it then differs too
    same = (tok.cpu() == want_tok).all(dim=1)
    assert same.float().mean() >= 0.6 and torch.allclose(p.cpu()[same], want_p[same], atol=2e-4)


@pytest.mark.parametrize("b,s,k", [(1, 15, 16), (9, 7, 4), (4, 3, 32), (2, 1, 1)])
def test_lattice_chain_walk_kernel(cu, b, s, k):
    g = torch.Generator().manual_seed(b * 100 + k)
    cand = torch.randint(0, 50000, (b, s, k), generator=g)
    tr = torch.randn(b, s, k, k, generator=g) * 3
    if k > 3 and s > 2:
        tr[0, 2, :, 1] = tr[0, 2, :, 3] = 50.0
    want_tok, want_p = ref.lattice_chain_walk(cand, tr)
    tok, p = cu.lattice_chain_walk(cand.cuda(), tr.cuda())
    assert torch.equal(tok.cpu(), want_tok) and torch.equal(p.cpu(), want_p)
    temps = torch.linspace(0.0, 1.6, b)
    uni = torch.rand(b, s, generator=g)
    want_tok, want_p = ref.lattice_chain_walk(cand, tr, temps, uni)
    tok, p = cu.lattice_chain_walk(cand.cuda(), tr.cuda(), temps.cuda(), uni.cuda())
    same = (tok.cpu() == want_tok).all(dim=1)
    assert same.float().mean() >= 0.6 and torch.allclose(p.cpu()[same], want_p[same], atol=2e-5)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("b,p,v,r", [(1, 6, 1000, 64), (5, 3, 4099, 256), (16, 6, 32000, 128), (2, 2, 300, 48)])
def test_markov_greedy_chain_kernel(cu, dtype, b, p, v, r):
    """Fused Markov correction + arg-max against the fp32 restatement; a step whose winner differs only through rounding of a
    near-tie would change everything after it, so agreement is asked of whole chains and must hold for nearly all of them."""
    g = torch.Generator().manual_seed(v + r)
    logits = torch.randn(b, p, v, generator=g) * 3
    w1 = (torch.randn(v, r, generator=g) / r ** 0.25).to(dtype)
    w2 = (torch.randn(v, r, generator=g) / r ** 0.25).to(dtype)
    first = torch.randint(0, v, (b,), generator=g)
    want = ref.markov_chain_propose(logits, w1, w2, first)
    got = cu.markov_greedy_chain(logits.cuda(), w1.cuda(), w2.cuda(), first.cuda()).cpu()
    assert got.shape == (b, p) and int(got.min()) >= 0 and int(got.max()) < v
    same = (got == want).all(dim=1)
    assert same.float().mean() >= 0.9
    # the correction matters: the uncorrected arg-max differs somewhere
    assert not torch.equal(want, logits.argmax(-1)) or b * p < 4
    # exact ties go to the lowest id
    lg = torch.zeros(1, 2, 64)
    lg[0, 0, 7] = lg[0, 0, 3] = 5.0
    z = torch.zeros(64, 32, dtype=dtype)
    tie = cu.markov_greedy_chain(lg.cuda(), z.cuda(), z.cuda(), torch.tensor([0]).cuda()).cpu()
    assert tie.tolist() == [[3, 0]]


@pytest.mark.parametrize("b,n,v,k", [(1, 8, 50, 2), (6, 40, 5000, 4), (3, 61, 32000, 8)])
def test_spec_accept_sampling_kernel(cu, b, n, v, k):
    """Device rejection sampling against the host restatement on random trees: peaked target rows so that paths of every
    length occur; a draw within rounding of a probability boundary may differ, so nearly all sequences must agree."""
    g = torch.Generator().manual_seed(n * k)
    tree, par = _random_tree(g, b, n, vocab=v)
    probs = torch.softmax(torch.randn(b, n, v, generator=g) * 2.0, dim=-1)
    for i in range(b):                                   # make some children likely under their parent's distribution
        for c in range(1, n):
            if c % 2:
                probs[i, par[i, c], tree[i, c]] += 2.0
        probs[i] /= probs[i].sum(-1, keepdim=True)
    max_path = 6
    agree = total = 0
    lens = set()
    for seed in range(4):
        u = torch.rand(b, max_path, k + 1, generator=torch.Generator().manual_seed(seed))
        want = ref.spec_accept_sampling(probs, tree, par, max_path, u)
        got = cu.spec_accept_sampling(probs.cuda(), tree.cuda(), par.cuda(), max_path, u.cuda())
        for i in range(b):
            m = int(want[1][i])
            lens.add(m)
            same = int(got[1][i]) == m and got[0][i, :m].cpu().tolist() == want[0][i, :m].tolist() and int(got[2][i]) == int(want[2][i])
            agree += int(same)
            total += 1
            assert 0 <= int(got[2][i]) < v and 1 <= int(got[1][i]) <= max_path
    assert agree >= total - 1 and len(lens) >= 2
    # a tree whose first child is certain, then a leaf: path root -> child, bonus from the child's row
    pr = torch.zeros(1, 2, 10)
    pr[0, 0, 4] = 1.0
    pr[0, 1, 7] = 1.0
    got = cu.spec_accept_sampling(pr.cuda(), torch.tensor([[0, 4]], dtype=torch.int32).cuda(), torch.tensor([[-1, 0]], dtype=torch.int32).cuda(), 4,
                                  torch.full((1, 4, 3), 0.5).cuda())
    assert got[1].tolist() == [2] and got[0][0, :2].tolist() == [0, 1] and got[2].tolist() == [7]
    # the only token with mass is a rejected candidate (u above its probability cannot happen at p = 1, so force p < 1 ... = residual fallback)
    pr = torch.zeros(1, 2, 10)
    pr[0, 0, 4] = 0.25
    pr[0, 0, 9] = 0.75
    pr[0, 1, 1] = 1.0
    got = cu.spec_accept_sampling(pr.cuda(), torch.tensor([[0, 4]], dtype=torch.int32).cuda(), torch.tensor([[-1, 0]], dtype=torch.int32).cuda(), 4,
                                  torch.full((1, 4, 3), 0.9).cuda())
    assert got[1].tolist() == [1] and got[2].tolist() == [9]


def test_hybrid_chain_commit_from_replay_data_on_gpu(cu):
    """Mamba2 / DeltaNet target on the GPU: a forced partial acceptance every round commits through the recorded recurrent-kernel
    inputs; the recurrent state afterwards equals the one left by the full-model replay of the same accepted tokens."""
    from tensorrt_edge_llm_b200 import AutoModel
    from tensorrt_edge_llm_b200.config import GdnConfig, MambaConfig, hybrid_nemotron_config, tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
    from tensorrt_edge_llm_b200.runtime.runner import ModelRunner
    from tensorrt_edge_llm_b200.runtime.speculative import EagleDecoder, SpecConfig
    dev = torch.device("cuda", 0)
    cfg = hybrid_nemotron_config(num_hidden_layers=8, vocab_size=1000, hidden_size=512, intermediate_size=1024, num_attention_heads=8,
                                 num_key_value_heads=2, head_dim=128, dtype="bfloat16", max_position_embeddings=1024,
                                 mamba=MambaConfig(num_heads=8, head_dim=64, d_state=128, n_groups=2, conv_kernel=4),
                                 gdn=GdnConfig(num_k_heads=2, num_v_heads=4, head_k_dim=128, head_v_dim=128, conv_kernel=4))
    model = AutoModel.from_config(cfg, random_init=0, device=dev)
    dcfg = tiny_llama_config(num_hidden_layers=1, hidden_size=512, intermediate_size=1024, num_attention_heads=8, num_key_value_heads=2,
                             head_dim=128, vocab_size=1000, dtype="bfloat16")
    dcfg.draft_type, dcfg.eagle3_target_hidden_size = "eagle3", 512
    draft = AutoModel.from_config(dcfg, random_init=2, device=dev)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (40, 75)]

    def run(use_record):
        kv = KVCacheManager(cfg, num_pages=16, page_size=64, max_seats=4, max_pages_per_seq=4, device=dev)
        dkv = KVCacheManager(dcfg, num_pages=16, page_size=64, max_seats=4, max_pages_per_seq=4, device=dev, num_layers=1)
        r = ModelRunner(model, kv, max_num_tokens=8192)
        r.use_cuda_graphs = False
        dec = EagleDecoder(r, draft, dkv, SpecConfig(draft_steps=3, top_k=1, verify_tokens=4, force_accept_len=2))
        dec.use_recurrent_replay = use_record
        dec.prefill([0, 1], prompts)
        out = [dec.round([0, 1]) for _ in range(5)]
        torch.cuda.synchronize()
        return out, [t.index_select(0, torch.tensor([0, 1], device=dev)).float().cpu() for t in kv.recurrent.pools()], dec.stats

    out_a, state_a, stats_a = run(True)
    out_b, state_b, stats_b = run(False)
    assert stats_a.recurrent_replays == stats_a.replays == 10 and stats_b.recurrent_replays == 0 and stats_b.replays == 10
    assert out_a == out_b
    for x, y in zip(state_a, state_b):
        assert torch.allclose(x, y, atol=2e-2, rtol=2e-2)
