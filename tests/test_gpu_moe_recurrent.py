"""GPU numerics of the MoE, recurrent-layer and sampling kernels against the fp32 PyTorch statements."""
import pytest
import torch

from tensorrt_edge_llm_b200.ops import build_step_meta
from tensorrt_edge_llm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cu():
    from tensorrt_edge_llm_b200.ops import cuda
    cuda.lib()
    return cuda


def _sync_check(cu):
    torch.cuda.synchronize()
    cu.Workspace.get(torch.device("cuda", 0)).check_status()


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("tokens,experts,top_k", [(1, 128, 8), (77, 128, 8), (300, 64, 6), (16, 8, 2)])
def test_moe_route_softmax(cu, tokens, experts, top_k):
    g = torch.Generator(device="cuda").manual_seed(0)
    logits = (2 * torch.randn(tokens, experts, device="cuda", generator=g)).bfloat16()
    for renorm in (True, False):
        w, idx = cu.moe_route_softmax_topk(logits, top_k, renorm)
        wr, idxr = ref.moe_route_softmax_topk(logits, top_k, renorm)
        assert torch.equal(idx, idxr)
        assert torch.allclose(w, wr, atol=1e-5, rtol=1e-4)
    _sync_check(cu)


def test_moe_route_sigmoid_groups(cu):
    g = torch.Generator(device="cuda").manual_seed(1)
    logits = torch.randn(33, 64, device="cuda", generator=g)
    bias = 0.1 * torch.randn(64, device="cuda", generator=g)
    w, idx = cu.moe_route_softmax_topk(logits, 6, True, bias=bias, sigmoid=True, n_group=8, topk_group=3, scaling=2.5)
    wr, idxr = ref.moe_route_sigmoid_group_topk(logits, bias, 6, 8, 3, True, 2.5)
    assert torch.equal(idx, idxr)
    assert torch.allclose(w, wr, atol=1e-5, rtol=1e-4)
    _sync_check(cu)


@pytest.mark.parametrize("tokens,experts,top_k,lo,hi", [(50, 16, 4, 0, 16), (300, 32, 8, 8, 16), (1, 128, 8, 0, 128)])
def test_moe_align_gather_combine(cu, tokens, experts, top_k, lo, hi):
    g = torch.Generator(device="cuda").manual_seed(2)
    h = 256
    idx = torch.stack([torch.randperm(experts, device="cuda", generator=g)[:top_k] for _ in range(tokens)]).to(torch.int32)
    w = torch.rand(tokens, top_k, device="cuda", generator=g)
    x = torch.randn(tokens, h, device="cuda", generator=g).bfloat16()
    ws = cu.moe_align(idx, experts, lo, hi)
    dst = ws.dst_row.view(tokens, top_k).long()
    local = (idx >= lo) & (idx < hi)
    assert torch.equal(dst >= 0, local)
    # every local slot has a unique row inside a tile owned by its expert; segments are 128-aligned
    rows = dst[local]
    assert rows.unique().numel() == rows.numel()
    te = ws.tile_expert.long()
    assert torch.equal(te[rows // 128], (idx[local] - lo).long())
    n_tiles = int(ws.counts.item()) // 128
    want_tiles = sum((int((idx == e).sum()) + 127) // 128 for e in range(lo, hi))
    assert n_tiles == want_tiles and torch.all(te[n_tiles:ws.max_tiles] < 0)
    # second half: rows in use per tile; they add up to the local slots and unused tiles hold none
    tile_rows = te[ws.max_tiles:]
    assert int(tile_rows.sum()) == int(local.sum()) and torch.all(tile_rows[n_tiles:] == 0) and int(tile_rows.max()) <= 128
    a = cu.moe_gather(x, ws, top_k, None)
    tok = torch.arange(tokens, device="cuda")[:, None].expand(tokens, top_k)[local]
    assert torch.equal(a[rows], x[tok])
    y = torch.randn(ws.rows_pad, h, device="cuda", generator=g).bfloat16()
    out = cu.moe_combine(y, ws, w)
    want = torch.zeros(tokens, h, device="cuda")
    want.index_add_(0, tok, y[rows].float() * w[local][:, None])
    assert _rel_err(out, want) < 4e-3
    _sync_check(cu)


@pytest.mark.parametrize("quant", ["bf16", "nvfp4"])
@pytest.mark.parametrize("tokens", [3, 200])
def test_moe_block_matches_reference(cu, quant, tokens):
    from tensorrt_edge_llm_b200.config import QuantConfig, qwen3_30b_a3b_config
    from tensorrt_edge_llm_b200.models.qwen3_moe import MoEBlock
    kw = dict(num_hidden_layers=1, hidden_size=512, moe_intermediate_size=256, num_experts=16, num_experts_per_tok=4)
    cfg = qwen3_30b_a3b_config(**kw)
    cfg.quant = QuantConfig(quant_type="nvfp4") if quant == "nvfp4" else QuantConfig()
    blk = MoEBlock(cfg, "model.layers.0.mlp").cuda()
    blk.random_init(torch.Generator().manual_seed(3), std=0.05)
    blk.finalize()
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(tokens, 512, device="cuda", generator=g).bfloat16()
    if quant == "nvfp4":
        blk.input_scale.fill_(float(x.abs().max()) / (6.0 * 448.0))
        blk.down_input_scale.fill_(0.5 / (6.0 * 448.0))
        blk._refresh_alpha()
    got = blk(x)
    want = blk._forward_reference(x)
    assert _rel_err(got, want) < (3e-2 if quant == "nvfp4" else 1e-2)
    _sync_check(cu)


@pytest.mark.parametrize("tokens", [5, 300])
def test_moe_fused_fc1_swiglu_matches_unfused(cu, tokens, monkeypatch):
    """Expert gate/up GEMM with SwiGLU + quantisation in its epilogue (interleaved expert rows) == GEMM then swiglu_quant."""
    from tensorrt_edge_llm_b200.config import QuantConfig, qwen3_30b_a3b_config
    from tensorrt_edge_llm_b200.models.qwen3_moe import MoEBlock
    kw = dict(num_hidden_layers=1, hidden_size=512, moe_intermediate_size=256, num_experts=16, num_experts_per_tok=4)
    cfg = qwen3_30b_a3b_config(**kw)
    cfg.quant = QuantConfig(quant_type="nvfp4")
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(tokens, 512, device="cuda", generator=g).bfloat16()
    outs = []
    for fused in (True, False):
        if fused:
            monkeypatch.setenv("TELB_MOE_SWIGLU_FUSION", "1")
        else:
            monkeypatch.delenv("TELB_MOE_SWIGLU_FUSION", raising=False)
        blk = MoEBlock(cfg, "model.layers.0.mlp").cuda()
        blk.random_init(torch.Generator().manual_seed(3), std=0.05)
        blk.finalize()
        assert blk._w13_interleaved == fused
        blk.input_scale.fill_(float(x.abs().max()) / (6.0 * 448.0))
        blk.down_input_scale.fill_(0.5 / (6.0 * 448.0))
        blk._refresh_alpha()
        outs.append(blk(x))
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    _sync_check(cu)


def _meta(q_lens, pasts, slots=None):
    table = torch.zeros(len(q_lens), 1, dtype=torch.int32)
    m = build_step_meta(q_lens, pasts, table, 64, slot_ids=slots)
    return m.to("cuda")


@pytest.mark.parametrize("q_lens,pasts", [([1, 1, 1], [5, 0, 9]), ([37, 1, 130], [0, 4, 64]), ([3], [0])])
def test_causal_conv1d(cu, q_lens, pasts):
    g = torch.Generator(device="cuda").manual_seed(5)
    c, w = 384, 4
    t = sum(q_lens)
    x = torch.randn(t, c, device="cuda", generator=g).bfloat16()
    weight = torch.randn(c, w, device="cuda", generator=g).bfloat16()
    bias = torch.randn(c, device="cuda", generator=g).bfloat16()
    slots = list(range(len(q_lens)))[::-1]
    meta = _meta(q_lens, pasts, slots)
    st = torch.randn(len(q_lens), c, w - 1, device="cuda", generator=g).bfloat16()
    st_ref = st.clone()
    y = cu.causal_conv1d(x, weight, bias, st, meta, True)
    yr = ref.causal_conv1d(x, weight, bias, st_ref, meta, True)
    assert _rel_err(y, yr) < 5e-3
    assert torch.equal(st, st_ref)
    _sync_check(cu)


@pytest.mark.parametrize("q_lens,pasts", [([1, 1], [7, 0]), ([20, 1, 5], [0, 3, 16]), ([300, 1, 517], [0, 9, 40]), ([256], [0])])
def test_ssm_scan(cu, q_lens, pasts):
    g = torch.Generator(device="cuda").manual_seed(6)
    nh, hd, ng, n = 8, 64, 2, 128
    t = sum(q_lens)
    x = torch.randn(t, nh, hd, device="cuda", generator=g).bfloat16()
    z = torch.randn(t, nh, hd, device="cuda", generator=g).bfloat16()
    dt = torch.randn(t, nh, device="cuda", generator=g).bfloat16()
    A = -torch.rand(nh, device="cuda", generator=g) - 0.5
    B = torch.randn(t, ng, n, device="cuda", generator=g).bfloat16()
    C = torch.randn(t, ng, n, device="cuda", generator=g).bfloat16()
    D = torch.randn(nh, device="cuda", generator=g)
    dtb = torch.randn(nh, device="cuda", generator=g)
    meta = _meta(q_lens, pasts)
    st = torch.randn(len(q_lens), nh, hd, n, device="cuda", generator=g)
    st_ref = st.clone()
    old, cu.SSD_TC_MIN_Q = cu.SSD_TC_MIN_Q, 1 << 30          # the sequential / segmented CUDA-core kernels
    try:
        y = cu.ssm_scan(x, dt, A, B, C, D, dtb, st, meta, z=z)
    finally:
        cu.SSD_TC_MIN_Q = old
    yr = ref.ssm_scan(x, dt, A, B, C, D, dtb, st_ref, meta, z=z)
    assert _rel_err(y, yr) < 6e-3
    assert _rel_err(st, st_ref) < 1e-4
    _sync_check(cu)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("q_lens,pasts,gate", [([256], [0], True), ([300, 1, 517], [0, 9, 40], True), ([128, 64, 129, 1000], [5, 0, 0, 64], False),
                                               ([2048, 77], [0, 300], True)])
def test_ssd_chunk_scan_tensor_cores(cu, q_lens, pasts, gate, dtype):
    """The chunked state-space-duality scan on tcgen05 against the sequential fp32 recurrence: ragged lengths (whole
    chunks, partial last chunks, a one-row sequence), carried-in states, with and without the gate.  The four products
    take 16-bit operands (the decay-masked scores, the rescaled inputs and the carried state are rounded to 16 bits), so
    the tolerance is that of 16-bit operands with fp32 accumulation."""
    g = torch.Generator(device="cuda").manual_seed(16)
    nh, hd, ng, n = 16, 64, 2, 128
    t = sum(q_lens)
    x = torch.randn(t, nh, hd, device="cuda", generator=g).to(dtype)
    z = torch.randn(t, nh, hd, device="cuda", generator=g).to(dtype) if gate else None
    dt = (torch.randn(t, nh, device="cuda", generator=g) - 1.0).to(dtype)
    A = -torch.rand(nh, device="cuda", generator=g) - 0.5
    B = (torch.randn(t, ng, n, device="cuda", generator=g) * 0.3).to(dtype)
    C = (torch.randn(t, ng, n, device="cuda", generator=g) * 0.3).to(dtype)
    D = torch.randn(nh, device="cuda", generator=g)
    dtb = torch.randn(nh, device="cuda", generator=g) * 0.5
    slots = list(range(len(q_lens)))[::-1]
    meta = _meta(q_lens, pasts, slots)
    st = torch.randn(len(q_lens), nh, hd, n, device="cuda", generator=g)
    st_ref = st.clone()
    assert max(q_lens) >= cu.SSD_TC_MIN_Q
    y = cu.ssm_scan(x, dt, A, B, C, D, dtb, st, meta, z=z, dt_limit=0.0)
    yr = ref.ssm_scan(x, dt, A, B, C, D, dtb, st_ref, meta, z=z)
    tol = 1.2e-2 if dtype == torch.bfloat16 else 3e-3
    assert _rel_err(y, yr) < tol, _rel_err(y, yr)
    assert _rel_err(st, st_ref) < tol, _rel_err(st, st_ref)
    # per sequence, so a short sequence cannot hide behind a long one
    r0 = 0
    for ql in q_lens:
        assert _rel_err(y[r0:r0 + ql], yr[r0:r0 + ql]) < 2 * tol
        r0 += ql
    _sync_check(cu)


@pytest.mark.parametrize("q_lens,pasts", [([1, 1], [7, 0]), ([12, 1], [0, 3])])
def test_gated_delta_rule(cu, q_lens, pasts):
    g = torch.Generator(device="cuda").manual_seed(7)
    hk, hv, kd, vd = 2, 4, 128, 128
    t = sum(q_lens)
    q = torch.randn(t, hk, kd, device="cuda", generator=g).bfloat16()
    k = torch.randn(t, hk, kd, device="cuda", generator=g).bfloat16()
    v = torch.randn(t, hv, vd, device="cuda", generator=g).bfloat16()
    a = torch.randn(t, hv, device="cuda", generator=g).bfloat16()
    b = torch.randn(t, hv, device="cuda", generator=g).bfloat16()
    A_log = torch.randn(hv, device="cuda", generator=g)
    dtb = torch.randn(hv, device="cuda", generator=g)
    meta = _meta(q_lens, pasts)
    st = 0.1 * torch.randn(len(q_lens), hv, kd, vd, device="cuda", generator=g)
    st_ref = st.clone()
    old, cu.GDN_TC_MIN_Q = cu.GDN_TC_MIN_Q, 1 << 30          # the sequential CUDA-core kernel
    try:
        o = cu.gated_delta_rule(q, k, v, a, b, A_log, dtb, st, meta)
    finally:
        cu.GDN_TC_MIN_Q = old
    orf = ref.gated_delta_rule(q, k, v, a, b, A_log, dtb, st_ref, meta)
    assert _rel_err(o, orf) < 6e-3
    assert _rel_err(st, st_ref) < 1e-4
    _sync_check(cu)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("q_lens,pasts", [([64], [0]), ([200, 1, 65], [0, 9, 40]), ([128, 33, 1000], [5, 0, 64]), ([2048], [0])])
def test_gdn_chunked_prefill_tensor_cores(cu, q_lens, pasts, dtype):
    """The 64-token chunked gated delta rule (tcgen05 products + per-column forward substitution) against the sequential
    fp32 recurrence: ragged lengths, carried-in states, two value heads per key head."""
    g = torch.Generator(device="cuda").manual_seed(17)
    hk, hv, kd, vd = 2, 4, 128, 128
    t = sum(q_lens)
    q = torch.randn(t, hk, kd, device="cuda", generator=g).to(dtype)
    k = torch.randn(t, hk, kd, device="cuda", generator=g).to(dtype)
    v = torch.randn(t, hv, vd, device="cuda", generator=g).to(dtype)
    a = torch.randn(t, hv, device="cuda", generator=g).to(dtype)
    b = torch.randn(t, hv, device="cuda", generator=g).to(dtype)
    A_log = torch.randn(hv, device="cuda", generator=g) * 0.5 - 1.0
    dtb = torch.randn(hv, device="cuda", generator=g) * 0.5
    slots = list(range(len(q_lens)))[::-1]
    meta = _meta(q_lens, pasts, slots)
    st = 0.1 * torch.randn(len(q_lens), hv, kd, vd, device="cuda", generator=g)
    st_ref = st.clone()
    assert max(q_lens) >= cu.GDN_TC_MIN_Q
    o = cu.gated_delta_rule(q, k, v, a, b, A_log, dtb, st, meta)
    orf = ref.gated_delta_rule(q, k, v, a, b, A_log, dtb, st_ref, meta)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert _rel_err(o, orf) < tol, _rel_err(o, orf)
    assert _rel_err(st, st_ref) < tol, _rel_err(st, st_ref)
    r0 = 0
    for ql in q_lens:
        assert _rel_err(o[r0:r0 + ql], orf[r0:r0 + ql]) < 2 * tol
        r0 += ql
    _sync_check(cu)


def test_sampling_ties_take_the_lowest_ids(cu):
    """Duplicated maxima in a batch that mixes greedy and sampled rows: a greedy row returns the lowest index of the
    maximum (what the arg-max kernel returns), on every run, and a top-k cut through a run of equal logits keeps the
    lowest ids."""
    g = torch.Generator(device="cuda").manual_seed(3)
    rows, vocab = 8, 151936
    logits = torch.randn(rows, vocab, device="cuda", generator=g).half()
    big = float(logits.float().max()) + 2.0
    ties = [[120000, 77, 9031, 150001], [5, 6, 7], [151935, 0], [42], [100, 50000, 60000, 70000, 80000], [3, 2, 1], [99999, 1234], [8, 80]]
    for r, ids in enumerate(ties):
        logits[r, ids] = big
    temp = torch.tensor([0.0, 0.8, 0.0, 1.0, 0.0, 0.0, 0.9, 0.0], device="cuda")
    top_k = torch.tensor([0, 2, 5, 1, 3, 1, 1, 40], device="cuda", dtype=torch.int32)
    top_p = torch.ones(rows, device="cuda")
    u = torch.full((rows,), 0.999, device="cuda")
    first = None
    for _ in range(5):
        got = cu.sample(logits, temp, top_k, top_p, u)
        first = got if first is None else first
        assert torch.equal(got, first)                         # arrival order plays no part
    for r, ids in enumerate(ties):
        if float(temp[r]) < 1e-3 or int(top_k[r]) == 1:
            assert int(first[r]) == min(ids)
        else:                                                   # row 1: top-2 of three equal maxima = the two lowest ids
            assert int(first[r]) in sorted(ids)[:int(top_k[r])]
    assert torch.equal(first[temp < 1e-3].long(), cu.argmax(logits)[temp < 1e-3].long())
    _sync_check(cu)


def test_sampling_kernel(cu):
    g = torch.Generator(device="cuda").manual_seed(8)
    rows, vocab = 48, 32000
    logits = (3 * torch.randn(rows, vocab, device="cuda", generator=g))
    temp = torch.tensor([0.0, 0.7, 1.0, 1.3] * (rows // 4), device="cuda")
    top_k = torch.tensor([0, 50, 1, 8, 1000, 20] * (rows // 6), device="cuda", dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.9, 0.5] * (rows // 3), device="cuda")
    u = torch.rand(rows, device="cuda", generator=g)
    for lg in (logits, logits.bfloat16()):
        got = cu.sample(lg, temp, top_k, top_p, u)
        kk = torch.where(top_k > 0, top_k, torch.full_like(top_k, 1024))
        want = ref.sample(lg, temp, kk, top_p, u)
        # cumulative sums differ in the last bits, so a draw that lands on a boundary may pick a neighbour
        assert (got == want).float().mean() >= 0.9
        greedy = temp < 1e-3
        assert torch.equal(got[greedy].long(), lg[greedy].float().argmax(-1))
        one = (top_k == 1)
        assert torch.equal(got[one].long(), lg[one].float().argmax(-1))
        for r in range(rows):                      # always inside the top-k set
            assert int(got[r]) in lg[r].float().topk(int(kk[r])).indices.tolist()
    # bitmask
    mask = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, (vocab + 31) // 32), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
    masked = cu.apply_token_bitmask(logits.clone(), mask)
    assert torch.equal(masked, ref.apply_token_bitmask(logits, mask))
    _sync_check(cu)


def test_hybrid_model_gpu_matches_cpu():
    from tensorrt_edge_llm_b200 import AutoModel
    from tensorrt_edge_llm_b200.config import GdnConfig, MambaConfig, hybrid_nemotron_config
    from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
    from tensorrt_edge_llm_b200.runtime.runner import ModelRunner
    cfg = hybrid_nemotron_config(num_hidden_layers=8, vocab_size=1000, hidden_size=512, intermediate_size=1024, num_attention_heads=8,
                                 num_key_value_heads=2, head_dim=128, dtype="bfloat16", max_position_embeddings=1024,
                                 mamba=MambaConfig(num_heads=8, head_dim=64, d_state=128, n_groups=2, conv_kernel=4),
                                 gdn=GdnConfig(num_k_heads=2, num_v_heads=4, head_k_dim=128, head_v_dim=128, conv_kernel=4))
    model = AutoModel.from_config(cfg, random_init=0)
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (40, 75)]

    def run(device):
        m = AutoModel.from_config(cfg)
        m.load_state_dict(sd)
        m = m.to(device)
        kv = KVCacheManager(cfg, num_pages=16, page_size=64, max_seats=4, max_pages_per_seq=4, device=device)
        r = ModelRunner(m, kv, max_num_tokens=8192)
        r.use_cuda_graphs = False
        a = r.prefill([0, 1], [s[:-2] for s in seqs]).float().cpu()
        b = r.step([0, 1], [[s[-2]] for s in seqs]).float().cpu()
        c = r.step([0, 1], [[s[-1]] for s in seqs]).float().cpu()
        return a, b, c

    cpu = run(torch.device("cpu"))
    gpu = run(torch.device("cuda", 0))
    for x, y in zip(gpu, cpu):
        assert _rel_err(x, y) < 5e-2
        assert torch.equal(x.argmax(-1), y.argmax(-1)) or _rel_err(x, y) < 2e-2


def test_int4_awq_linear_gpu(cu):
    from tensorrt_edge_llm_b200.models.linear import Int4AwqLinear
    g = torch.Generator().manual_seed(9)
    lin = Int4AwqLinear(512, [384], group_size=128, dtype=torch.bfloat16)
    lin.quantize_from([torch.randn(384, 512, generator=g) * 0.05])
    x = torch.randn(70, 512, generator=g).bfloat16()
    want = lin(x).float()
    got = lin.cuda()(x.cuda()).float().cpu()
    assert _rel_err(got, want) < 1e-2
    _sync_check(cu)


@pytest.mark.parametrize("rows,hidden", [(5, 1024), (33, 1152), (2, 8192)])
def test_layernorm(cu, rows, hidden):
    g = torch.Generator(device="cuda").manual_seed(10)
    x = (torch.randn(rows, hidden, device="cuda", generator=g) * 2 + 0.5).bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).bfloat16()
    b = (0.1 * torch.randn(hidden, device="cuda", generator=g)).bfloat16()
    assert _rel_err(cu.layernorm(x, w, b, 1e-5), ref.layernorm(x, w, b, 1e-5)) < 4e-3
    assert _rel_err(cu.layernorm(x, w, None, 1e-5), ref.layernorm(x, w, None, 1e-5)) < 4e-3
    _sync_check(cu)


def test_vision_encoder_gpu_matches_cpu(cu):
    from tensorrt_edge_llm_b200.models.vit import VisionConfig, VisionEncoder
    cfg = VisionConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512, patch_size=4, image_size=64,
                       out_hidden_size=512, dtype="bfloat16")
    enc = VisionEncoder(cfg).random_init(0, std=0.05)
    patches = VisionEncoder.patchify(torch.randn(2, 3, 64, 64, generator=torch.Generator().manual_seed(3)), 4)      # 256 patches each
    want = enc(patches).float()
    got = enc.cuda()(patches.cuda()).float().cpu()
    assert got.shape == (2 * 64, 512) and _rel_err(got, want) < 3e-2
    x = torch.randn(40, 64, generator=torch.Generator().manual_seed(4)).bfloat16()
    for approx in (False, True):
        assert _rel_err(cu.gelu(x.cuda(), approx).cpu(), torch.nn.functional.gelu(x.float(), approximate="tanh" if approx else "none")) < 5e-3
    _sync_check(cu)


@pytest.mark.parametrize("tanh", [True, False])
def test_geglu(cu, tanh):
    from tensorrt_edge_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(12)
    x = (torch.randn(37, 2 * 264, device="cuda", generator=g) * 1.5).bfloat16()
    want = ops.geglu(x.cpu(), tanh).float()
    got = cu.geglu(x, tanh).float().cpu()
    assert (got - want).abs().max() < 2e-2 * want.abs().max()
    _sync_check(cu)


def test_audio_encoder_gpu_matches_cpu(cu):
    from tensorrt_edge_llm_b200.models.audio import AudioConfig, AudioEncoder
    cfg = AudioConfig(n_mels=64, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512, max_source_positions=100,
                      avg_pool=2, out_hidden_size=256, dtype="bfloat16")
    enc = AudioEncoder(cfg).random_init(0, std=0.05)
    mel = torch.randn(2, 64, 200, generator=torch.Generator().manual_seed(3))
    want = enc(mel).float()
    got = enc.to("cuda")(mel.cuda()).float().cpu()
    assert got.shape == (100, 256)
    assert (got - want).abs().max() < 0.05 * max(want.abs().max().item(), 1.0)
    _sync_check(cu)
