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
