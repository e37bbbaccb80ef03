"""Fused tensor-parallel prefill path on one GPU: GEMM with a reduce-scatter epilogue, the
reduce + add + RMSNorm (+NVFP4) + all-gather kernel and the GEMM with an all-gather prologue.
Two ranks are emulated with two sets of buffers in one process; the flags each kernel would wait
for are set by the host beforehand, so no kernel ever waits for another launch."""
import ctypes

import pytest
import torch

from tensorrt_edge_llm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cu():
    from tensorrt_edge_llm_b200.ops import cuda
    cuda.lib()
    return cuda


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _table(tensors, offset=0):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() + offset for t in tensors])


@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("m", [24, 64, 300, 1024])
def test_rs_norm_ag_two_emulated_ranks(cu, quant, m):
    # m <= 128 runs the decode-size (swapped-operand, cluster split-K) GEMM with the same epilogue / prologue
    g = torch.Generator(device="cuda").manual_seed(m)
    world, h, ks, n2 = 2, 512, 256, 768
    rpr = (m + world - 1) // world
    x = (torch.randn(m, world * ks, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(h, world * ks, device="cuda", generator=g) * 0.05).bfloat16()
    resid = torch.randn(m, h, device="cuda", generator=g).bfloat16()
    gamma = (1 + 0.1 * torch.randn(h, device="cuda", generator=g)).bfloat16()
    w2 = (torch.randn(n2, h, device="cuda", generator=g) * 0.05).bfloat16()
    partial = [torch.zeros(world * rpr * h, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    gy = [torch.zeros(m, h, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    L = cu.lib()
    L.telb_nvfp4_sf_bytes.restype = ctypes.c_longlong
    sfb = int(L.telb_nvfp4_sf_bytes(ctypes.c_longlong(m), ctypes.c_int(h)))
    gxq = [torch.zeros(m, h // 2, device="cuda", dtype=torch.uint8) for _ in range(world)]
    gsf = [torch.zeros(sfb, device="cuda", dtype=torch.uint8) for _ in range(world)]
    flags = [torch.ones(16, device="cuda", dtype=torch.int32) for _ in range(world)]     # epoch 1 already "published"
    epoch = [torch.zeros(1, device="cuda", dtype=torch.int32) for _ in range(world)]
    ticket = [torch.zeros(1, device="cuda", dtype=torch.int32) for _ in range(world)]
    qscale = torch.tensor(4.0 / (6.0 * 448.0), device="cuda")
    ws = cu.Workspace.get(x.device)
    # 1. both ranks' row-parallel GEMMs scatter their partial rows
    for r in range(world):
        f = cu.GemmFusion()
        for d in range(world):
            f.rs_out[d] = partial[d].data_ptr()
        f.rs_world, f.rs_rank, f.rs_rows_per_rank = world, r, rpr
        cu.gemm_fused(x[:, r * ks:(r + 1) * ks].contiguous(), w[:, r * ks:(r + 1) * ks].contiguous(), f)
    parts = [x[:, r * ks:(r + 1) * ks].float() @ w[:, r * ks:(r + 1) * ks].float().t() for r in range(world)]
    for d in range(world):
        rows_d = max(0, min(rpr, m - d * rpr))
        buf = partial[d].view(world, rpr, h)
        for r in range(world):
            assert _rel_err(buf[r, :rows_d], parts[r][d * rpr:d * rpr + rows_d]) < 6e-3
    # 2. each owner reduces, adds its residual rows, normalises and pushes to both gather buffers
    res_out = []
    for r in range(world):
        rows_r = max(0, min(rpr, m - r * rpr))
        ro = torch.empty(rows_r, h, device="cuda", dtype=torch.bfloat16)
        cu._check(L.telb_rs_add_rmsnorm_ag(
            cu._p(partial[r]), _table(flags), _table(flags, 32), cu._p(epoch[r]), cu._p(ticket[r]), cu._p(resid), 1, cu._p(gamma),
            cu._p(ro), None if quant else _table(gy), _table(gxq) if quant else None, _table(gsf) if quant else None,
            cu._p(qscale) if quant else None, r, world, m, rpr, h, ctypes.c_float(1e-6), 0, 1, cu._p(ws.status), 0, 0, cu._stream()), "rs")
        res_out.append(ro)
    torch.cuda.synchronize()
    ws.check_status()
    summed = sum(p.bfloat16().float() for p in parts).bfloat16()
    want_y, want_res = ref.add_rmsnorm(summed, resid, gamma, 1e-6)
    got_res = torch.cat(res_out)
    assert _rel_err(got_res, want_res) < 6e-3
    assert [int(e) for e in epoch] == [1, 1] and [int(t) for t in ticket] == [0, 0]
    assert all(int(f[8 + r]) == 1 for f in flags for r in range(world))
    # 3. the next (column-parallel) GEMM reads the gathered rows, waiting on the gather flags in its producer
    f = cu.GemmFusion()
    f.ag_flags, f.ag_epoch, f.ag_world, f.ag_rows_per_rank = flags[0].data_ptr() + 32, epoch[0].data_ptr(), world, rpr
    if quant:
        assert torch.equal(gxq[0], gxq[1]) and torch.equal(gsf[0], gsf[1])
        w2q, w2sf, w2gs = ref.nvfp4_quantize(w2.float())
        w2_atoms = cu.nvfp4_swizzle_scales(w2sf.cuda())
        alpha = (w2gs.cuda() * qscale).expand(n2).contiguous()
        acts = cu.QuantActs(gxq[0], gsf[0], (m, h), torch.bfloat16)
        got = cu.gemm_fused(acts, w2q.cuda(), f, w_sf=w2_atoms, alpha=alpha)
        plain = cu.gemm_nvfp4(gxq[0], gsf[0], w2q.cuda(), w2_atoms, alpha, torch.bfloat16, mode=1 if m > 128 else 0)
        assert torch.equal(got, plain)
        y_dq = ref.nvfp4_act_qdq(want_y.float(), qscale)
        w_dq = ref.nvfp4_dequantize(w2q.cuda(), w2sf.cuda(), w2gs.cuda())
        assert _rel_err(got, y_dq @ w_dq.float().t()) < 3e-2
    else:
        assert torch.equal(gy[0], gy[1])
        assert _rel_err(gy[0], want_y) < 8e-3
        got = cu.gemm_fused(gy[0], w2, f)
        assert torch.equal(got, cu.gemm(gy[0], w2, mode=1 if m > 128 else 0))
    torch.cuda.synchronize()
    ws.check_status()


def test_ep_all_to_all_two_emulated_ranks(cu):
    """Dispatch → align / gather / grouped GEMM → return → weighted combine, two ranks emulated on one GPU."""
    g = torch.Generator(device="cuda").manual_seed(5)
    world, h, top_k, experts, cap_tokens = 2, 256, 2, 8, 200
    epr, cap = experts // world, cap_tokens * top_k
    t_local = [150, 97]
    x = [torch.randn(t, h, device="cuda", generator=g).bfloat16() for t in t_local]
    idx = [torch.stack([torch.randperm(experts, device="cuda", generator=g)[:top_k] for _ in range(t)]).to(torch.int32) for t in t_local]
    w = [torch.rand(t, top_k, device="cuda", generator=g) for t in t_local]
    wexp = [(torch.randn(epr * h, h, device="cuda", generator=g) * 0.05).bfloat16() for _ in range(world)]     # per rank [epr * N, K]
    recv_rows = [torch.zeros(world * cap * h, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    recv_ids = [torch.full((world * cap,), -1, device="cuda", dtype=torch.int32) for _ in range(world)]
    comb = [torch.zeros(cap * h, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    flags = [torch.ones(16, device="cuda", dtype=torch.int32) for _ in range(world)]      # epoch 1 already "published"
    epoch = [torch.zeros(2, device="cuda", dtype=torch.int32) for _ in range(world)]
    ticket = [torch.zeros(2, device="cuda", dtype=torch.int32) for _ in range(world)]
    L, ws0 = cu.lib(), cu.Workspace.get(torch.device("cuda", 0))
    tables = (_table(recv_rows), _table(recv_ids), _table(comb), _table(flags))
    for r in range(world):
        cu._check(L.telb_ep_dispatch(cu._p(x[r]), cu._p(idx[r]), *tables, r, world, t_local[r], top_k, h, epr, cap,
                                     ctypes.c_void_p(epoch[r].data_ptr()), ctypes.c_void_p(ticket[r].data_ptr()), cu._stream()), "dispatch")
    for r in range(world):
        cu._check(L.telb_ep_wait(cu._p(flags[r]), 0, world, ctypes.c_void_p(epoch[r].data_ptr()), cu._p(ws0.status), cu._stream()), "wait")
    torch.cuda.synchronize()
    for r in range(world):      # every slot of every source carries this rank's local expert id or -1
        for s in range(world):
            ids = recv_ids[r].view(world, cap)[s, :t_local[s] * top_k]
            want = torch.where(idx[s].view(-1) // epr == r, idx[s].view(-1) % epr, torch.full_like(idx[s].view(-1), -1))
            assert torch.equal(ids, want)
    for r in range(world):
        ws = cu.moe_align(recv_ids[r].view(-1, 1), epr, 0, epr)
        a = cu.moe_gather(recv_rows[r].view(world * cap, h), ws, 1, None)
        y = cu.gemm_grouped(a, wexp[r], ws, epr)
        cu._check(L.telb_ep_return(cu._p(y), cu._p(ws.dst_row), *tables, r, world, cap, h, ctypes.c_void_p(epoch[r].data_ptr() + 4),
                                   ctypes.c_void_p(ticket[r].data_ptr() + 4), cu._stream()), "return")
    from tensorrt_edge_llm_b200.parallel.fused import _Rows
    arange = torch.arange(cap, device="cuda", dtype=torch.int32)
    for r in range(world):
        cu._check(L.telb_ep_wait(cu._p(flags[r]), 1, world, ctypes.c_void_p(epoch[r].data_ptr() + 4), cu._p(ws0.status), cu._stream()), "wait")
        out = cu.moe_combine(comb[r].view(cap, h), _Rows(arange), w[r])
        want = torch.zeros(t_local[r], h, device="cuda")
        for k in range(top_k):
            e = idx[r][:, k].long()
            wk = torch.stack([wexp[int(ee) // epr].view(epr, h, h)[int(ee) % epr] for ee in e]).float()      # [T, N, K]
            want += w[r][:, k, None] * torch.einsum("tk,tnk->tn", x[r].float(), wk).bfloat16().float()
        assert _rel_err(out, want) < 1e-2
    torch.cuda.synchronize()
    assert [e.tolist() for e in epoch] == [[1, 1], [1, 1]] and all(t.tolist() == [0, 0] for t in ticket)
    # a shorter step after a longer one: the whole segment of the slot stride is rewritten, so no stale id survives
    cu._check(L.telb_ep_dispatch(cu._p(x[0][:10]), cu._p(idx[0][:10].contiguous()), *tables, 0, world, 10, top_k, h, epr, cap,
                                 ctypes.c_void_p(epoch[0].data_ptr()), ctypes.c_void_p(ticket[0].data_ptr()), cu._stream()), "dispatch")
    torch.cuda.synchronize()
    for r in range(world):
        assert int((recv_ids[r].view(world, cap)[0, 10 * top_k:] != -1).sum()) == 0
    ws0.check_status()


def test_argmax_merge_two_emulated_ranks(cu):
    """Vocabulary-sharded greedy pick: each "rank" publishes its shard's best (value, global id) per row into both tables;
    the rank that runs last sees every candidate and must return the arg-max of the concatenated logits (lowest id on ties)."""
    g = torch.Generator(device="cuda").manual_seed(21)
    world, rows, vloc, max_rows = 2, 37, 5000, 1024
    full = torch.randn(rows, world * vloc, device="cuda", generator=g).half()
    full[0, 17] = full[0, vloc + 3] = 9.0                 # tie across shards: id 17 wins
    full[1, vloc + 100] = full[1, vloc + 4000] = 9.5      # tie inside shard 1: the lower id wins
    keys = [torch.zeros(2 * 8 * max_rows, device="cuda", dtype=torch.int64) for _ in range(world)]
    flags = [torch.ones(16, device="cuda", dtype=torch.int32) for _ in range(world)]          # epoch 1 already "published"
    epoch = [torch.zeros(1, device="cuda", dtype=torch.int32) for _ in range(world)]
    outs = [torch.full((rows,), -1, device="cuda", dtype=torch.int32) for _ in range(world)]
    ws = cu.Workspace.get(full.device)
    L = cu.lib()
    for r in (1, 0):                                        # rank 0 runs last and sees both shards' candidates
        shard = full[:, r * vloc:(r + 1) * vloc]            # a strided view: row pitch = world * vloc
        local = cu.argmax(shard)
        cu._check(L.telb_argmax_merge(cu._p(shard), ctypes.c_longlong(shard.stride(0)), cu._p(local), _table(keys), _table(flags),
                                      cu._p(epoch[r]), cu._p(outs[r]), r, world, rows, max_rows, vloc, 0, cu._p(ws.status), cu._stream()),
                  "argmax_merge")
    torch.cuda.synchronize()
    ws.check_status()
    want = (full.float() == full.float().max(-1, keepdim=True).values).to(torch.int32).argmax(-1).to(torch.int32)
    assert torch.equal(outs[0], want)
    assert int(outs[0][0]) == 17 and int(outs[0][1]) == vloc + 100
    assert [int(e) for e in epoch] == [1, 1]
