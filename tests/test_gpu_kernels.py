"""Numerics of the sm_100a kernels against the plain-PyTorch fp32 statements of the same ops."""
import math

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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,hidden", [(1, 4096), (7, 2048), (64, 4096), (3, 256), (5, 12288)])
def test_rmsnorm(cu, dtype, rows, hidden):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, hidden, device="cuda", generator=g).to(dtype)
    r = torch.randn(rows, hidden, device="cuda", generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).to(dtype)
    y = cu.rmsnorm(x, w, 1e-6)
    assert _rel_err(y, ref.rmsnorm(x, w, 1e-6)) < 2e-3
    y2, res = cu.add_rmsnorm(x, r, w, 1e-6)
    y2r, resr = ref.add_rmsnorm(x, r, w, 1e-6)
    assert torch.equal(res, resr)
    assert _rel_err(y2, y2r) < 2e-3
    _sync_check(cu)


def test_swiglu_relu2_embedding_argmax(cu):
    g = torch.Generator(device="cuda").manual_seed(1)
    gu = torch.randn(33, 2 * 1536, device="cuda", generator=g).bfloat16()
    assert _rel_err(cu.swiglu(gu), ref.swiglu(gu)) < 4e-3
    x = torch.randn(9, 1024, device="cuda", generator=g).bfloat16()
    assert _rel_err(cu.relu2(x), ref.relu2(x)) < 4e-3
    table = torch.randn(1000, 512, device="cuda", generator=g).bfloat16()
    ids = torch.randint(0, 1000, (77,), device="cuda", generator=g, dtype=torch.int32)
    assert torch.equal(cu.embedding(ids, table), table[ids.long()])
    logits = torch.randn(5, 151936, device="cuda", generator=g).bfloat16()
    assert torch.equal(cu.argmax(logits).long(), logits.float().argmax(-1))
    lf = torch.randn(3, 32000, device="cuda", generator=g)
    assert torch.equal(cu.argmax(lf).long(), lf.argmax(-1))
    z = torch.randn(4, 1024, device="cuda", generator=g).bfloat16()
    w = torch.randn(1024, device="cuda", generator=g).bfloat16()
    assert _rel_err(cu.gated_group_rmsnorm(x[:4], z, w, 8, 1e-5), ref.gated_group_rmsnorm(x[:4], z, w, 8, 1e-5)) < 4e-3
    _sync_check(cu)


GEMM_SHAPES = [
    # (M, N, K)  large-M layout
    (256, 512, 256), (1024, 6144, 4096), (300, 1000, 512), (129, 320, 192), (4096, 4096, 4096),
    # small-M (swapped, split-K) layout
    (1, 4096, 4096), (8, 6144, 4096), (16, 4096, 12288), (33, 1024, 512), (64, 24576, 4096), (100, 4096, 4096),
    (7, 151936, 4096),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
def test_gemm(cu, dtype, m, n, k):
    if dtype == torch.float16 and (m, n, k) not in [(256, 512, 256), (8, 6144, 4096), (129, 320, 192)]:
        pytest.skip("fp16 covered on a subset")
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n)
    x = (torch.randn(m, k, device="cuda", generator=g) * 0.5).to(dtype)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(dtype)
    y = cu.gemm(x, w)
    torch.cuda.synchronize()
    yr = x.float() @ w.float().t()
    assert _rel_err(y, yr) < 6e-3, f"rel err {_rel_err(y, yr)}"
    _sync_check(cu)


def test_gemm_epilogue_and_modes(cu):
    g = torch.Generator(device="cuda").manual_seed(5)
    for m, mode in [(48, 2), (48, 1), (200, 1), (200, 2)]:
        n, k = 768, 1024
        x = (torch.randn(m, k, device="cuda", generator=g) * 0.5).bfloat16()
        w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
        b = torch.randn(n, device="cuda", generator=g).bfloat16()
        a = torch.rand(n, device="cuda", generator=g) + 0.5
        r = torch.randn(m, n, device="cuda", generator=g).bfloat16()
        y = cu.gemm(x, w, bias=b, alpha=a, residual=r, mode=mode)
        yr = (x.float() @ w.float().t()) * a + b.float() + r.float()
        assert _rel_err(y, yr) < 6e-3, (m, mode, _rel_err(y, yr))
    # repeated split-K launches reuse the self-resetting tile counters
    x = (torch.randn(4, 4096, device="cuda", generator=g)).bfloat16()
    w = (torch.randn(512, 4096, device="cuda", generator=g) * 0.05).bfloat16()
    yr = x.float() @ w.float().t()
    for s in (1, 4, 16, 4):
        assert _rel_err(cu.gemm(x, w, splits=s), yr) < 6e-3
    _sync_check(cu)


def _paged_setup(q_lens, past_lens, hq, hkv, d, page, dtype, seed=0, extra_pages=3):
    g = torch.Generator(device="cuda").manual_seed(seed)
    n = len(q_lens)
    max_pages = max((q + p + page - 1) // page for q, p in zip(q_lens, past_lens)) + 1
    total_pages = n * max_pages + extra_pages
    perm = torch.randperm(total_pages, generator=torch.Generator().manual_seed(seed))
    table = torch.full((n, max_pages), -1, dtype=torch.int32)
    k = 0
    for s in range(n):
        need = (q_lens[s] + past_lens[s] + page - 1) // page
        table[s, :need] = perm[k:k + need].to(torch.int32)
        k += need
    kv = (torch.randn(total_pages, 2, hkv, page, d, device="cuda", generator=g)).to(dtype)
    meta = build_step_meta(q_lens, past_lens, table, page, device="cuda")
    t = sum(q_lens)
    q = torch.randn(t, hq, d, device="cuda", generator=g).to(dtype)
    return q, kv, meta


ATTN_CASES = [
    # q_lens, past_lens, hq, hkv, d, page
    ([1], [100], 32, 8, 128, 64),
    ([1, 1, 1], [5, 64, 700], 32, 8, 128, 64),
    ([128], [0], 32, 8, 128, 64),
    ([200, 37], [0, 91], 8, 2, 128, 64),
    ([64, 1, 300], [64, 1000, 17], 16, 4, 128, 64),
    ([70], [130], 4, 4, 128, 64),
    ([33, 1], [10, 200], 8, 1, 64, 64),
    ([150], [50], 32, 8, 128, 128),
    ([70, 33], [130, 10], 8, 2, 256, 64),           # 256-wide heads (Gemma family)
    ([1, 1, 1], [300, 77, 1000], 8, 4, 256, 64),
    ([260], [0], 4, 1, 256, 128),
]


@pytest.mark.parametrize("case", ATTN_CASES)
def test_paged_attention(cu, case):
    q_lens, past_lens, hq, hkv, d, page = case
    q, kv, meta = _paged_setup(q_lens, past_lens, hq, hkv, d, page, torch.bfloat16, seed=len(q_lens))
    scale = d ** -0.5
    out = cu.paged_attention(q, kv, meta, scale, kernel="tile")
    torch.cuda.synchronize()
    outr = ref.paged_attention(q, kv, meta, scale)
    assert _rel_err(out, outr) < 1.5e-2, _rel_err(out, outr)
    if d == 256:                                     # split-KV merge and sliding window on the wide-head instantiation
        assert _rel_err(cu.paged_attention(q, kv, meta, scale, kernel="tile", splits=3), outr) < 1.5e-2
        outw = cu.paged_attention(q, kv, meta, scale, sliding_window=64)
        assert _rel_err(outw, ref.paged_attention(q, kv, meta, scale, sliding_window=64)) < 1.5e-2
    _sync_check(cu)


DECODE_CASES = [
    # q_lens, past_lens, hq, hkv, page
    ([1], [100], 32, 8, 64), ([1, 1, 1], [5, 64, 700], 32, 8, 64), ([1] * 9, [0, 1, 63, 64, 127, 128, 129, 1000, 2047], 32, 8, 64),
    ([2, 1, 4], [10, 300, 77], 16, 4, 64), ([1, 1], [200, 31], 8, 8, 64), ([1, 1], [500, 90], 16, 1, 64),
    ([1, 3], [150, 260], 32, 8, 128), ([1, 1], [900, 333], 4, 2, 64),
]


@pytest.mark.parametrize("case", DECODE_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_attention_decode_kernel(cu, case, dtype):
    q_lens, past_lens, hq, hkv, page = case
    q, kv, meta = _paged_setup(q_lens, past_lens, hq, hkv, 128, page, dtype, seed=sum(past_lens))
    scale = 128 ** -0.5
    outr = ref.paged_attention(q, kv, meta, scale)
    for s in (1, 3):
        out = cu.paged_attention(q, kv, meta, scale, kernel="decode", splits=s)
        torch.cuda.synchronize()
        assert _rel_err(out, outr) < 1.5e-2, (s, _rel_err(out, outr))
    outw = cu.paged_attention(q, kv, meta, scale, kernel="decode", sliding_window=100)
    assert _rel_err(outw, ref.paged_attention(q, kv, meta, scale, sliding_window=100)) < 1.5e-2
    _sync_check(cu)


def _sf_rows_index(rows, k):
    """Byte offsets of the scales of rows [0, rows) in the 512-byte atom layout (padding rows hold anything)."""
    r = torch.arange(rows).view(-1, 1)
    kb = torch.arange(k // 16).view(1, -1)
    k64 = (k + 255) // 256 * 4
    off = ((r >> 7) * k64 + (kb >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (kb & 3)
    return off.reshape(-1).cuda()


@pytest.mark.parametrize("case", DECODE_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_attention_decode_nvfp4_output(cu, case, dtype):
    """The decode kernel's NVFP4 epilogue (and the quantising split merge) equal the 16-bit output passed through
    the stand-alone quantiser, bit for bit."""
    q_lens, past_lens, hq, hkv, page = case
    q, kv, meta = _paged_setup(q_lens, past_lens, hq, hkv, 128, page, dtype, seed=sum(past_lens))
    scale = 128 ** -0.5
    gs = torch.tensor(0.004, device="cuda")
    for s in (1, 3):
        out = cu.paged_attention(q, kv, meta, scale, kernel="decode", splits=s)
        xq_ref, sf_ref = cu.nvfp4_quantize(out.reshape(out.shape[0], -1), gs)
        qa = cu.paged_attention_quant(q, kv, meta, scale, None, gs, splits=s)
        torch.cuda.synchronize()
        assert qa.shape == (q.shape[0], hq * 128)
        assert torch.equal(qa.xq, xq_ref), s
        assert torch.equal(qa.sf[_sf_rows_index(q.shape[0], hq * 128)], sf_ref[_sf_rows_index(q.shape[0], hq * 128)]), s
    _sync_check(cu)


@pytest.mark.parametrize("kernel,case", [("tile", ([200, 37], [0, 91], 8, 2, 128, 64)), ("tile", ([33, 1], [10, 200], 8, 1, 64, 64)),
                                         ("decode", ([1, 1, 1], [5, 64, 700], 32, 8, 128, 64)), ("decode", ([2, 1, 4], [10, 300, 77], 16, 4, 128, 64))])
def test_paged_attention_sinks(cu, kernel, case):
    """Per-head sink logits (one extra softmax column without a value row) in both kernels, with and without KV splits."""
    q_lens, past_lens, hq, hkv, d, page = case
    q, kv, meta = _paged_setup(q_lens, past_lens, hq, hkv, d, page, torch.bfloat16, seed=5)
    scale = d ** -0.5
    sinks = torch.linspace(-3.0, 6.0, hq, device="cuda")
    outr = ref.paged_attention(q, kv, meta, scale, sinks=sinks)
    assert _rel_err(outr, ref.paged_attention(q, kv, meta, scale)) > 0.05          # the sinks matter in this case
    for s in (1, 3):
        out = cu.paged_attention(q, kv, meta, scale, sinks=sinks, kernel=kernel, splits=s)
        torch.cuda.synchronize()
        assert _rel_err(out, outr) < 1.5e-2, (s, _rel_err(out, outr))
    _sync_check(cu)


def test_paged_attention_skip_softmax_tile_vote(cu):
    """BLASST tile vote: with a threshold, tiles whose scores all sit far below the running maximum are dropped (counted by the
    kernel) and the result stays within the bound the threshold promises; without one (-inf) the kernel is bit-identical to
    the dense run and drops nothing."""
    q_lens, past_lens, hq, hkv, d, page = [512, 300], [1024, 0], 8, 2, 128, 64
    q, kv, meta = _paged_setup(q_lens, past_lens, hq, hkv, d, page, torch.bfloat16, seed=11)
    # "A-shaped" attention: the first 64 cached tokens and the most recent ones carry the weight, the far field is weak
    kv[:, 0] *= 0.05
    table = meta.page_table
    for s_ in range(2):
        first = int(table[s_, 0])
        kv[first, 0] *= 400.0
    scale = d ** -0.5
    dense = cu.paged_attention(q, kv, meta, scale, kernel="tile", splits=1)
    stats = torch.zeros(2, dtype=torch.int32, device="cuda")
    off = torch.full((2,), float("-inf"), device="cuda")
    same = cu.paged_attention(q, kv, meta, scale, kernel="tile", splits=1, skip_thr=off, skip_stats=stats)
    torch.cuda.synchronize()
    assert torch.equal(same, dense) and int(stats[1]) == 0 and int(stats[0]) > 0
    lam = 1e-3
    thr = torch.full((2,), float(torch.log2(torch.tensor(lam))), device="cuda")
    stats.zero_()
    got = cu.paged_attention(q, kv, meta, scale, kernel="tile", splits=1, skip_thr=thr, skip_stats=stats)
    torch.cuda.synchronize()
    tiles, skipped = int(stats[0]), int(stats[1])
    assert skipped > 0.2 * tiles, (tiles, skipped)
    # every dropped weight is below lambda relative to a normaliser of at least one: the error is a small multiple of lambda * L * |V|
    assert _rel_err(got, dense) < 2e-2, _rel_err(got, dense)
    assert not torch.isnan(got.float()).any()
    # per-sequence thresholds: a dense sequence next to a skipping one is bit-identical to its dense result
    mixed = torch.tensor([float("-inf"), float(thr[0])], device="cuda")
    got2 = cu.paged_attention(q, kv, meta, scale, kernel="tile", splits=1, skip_thr=mixed)
    assert torch.equal(got2[:512], dense[:512])
    _sync_check(cu)


def test_paged_attention_splits_window_tree(cu):
    q, kv, meta = _paged_setup([1, 1], [900, 333], 32, 8, 128, 64, torch.bfloat16, seed=9)
    scale = 128 ** -0.5
    outr = ref.paged_attention(q, kv, meta, scale)
    for s in (1, 2, 5, 16):
        assert _rel_err(cu.paged_attention(q, kv, meta, scale, splits=s, kernel="tile"), outr) < 1.5e-2, s
    q, kv, meta = _paged_setup([96, 1], [200, 500], 8, 2, 128, 64, torch.float16, seed=3)
    outr = ref.paged_attention(q, kv, meta, scale, sliding_window=128)
    assert _rel_err(cu.paged_attention(q, kv, meta, scale, sliding_window=128), outr) < 1.5e-2
    # speculative tree: 12 new rows per sequence with a random ancestor mask (row sees itself)
    q, kv, meta = _paged_setup([12, 12], [77, 300], 32, 8, 128, 64, torch.bfloat16, seed=4)
    gm = torch.Generator().manual_seed(0)
    bits = (torch.rand(24, 12, generator=gm) < 0.5) | torch.eye(12).repeat(2, 1).bool()
    bits = torch.tril(bits.view(2, 12, 12)).view(24, 12)
    words = (bits.long() << torch.arange(12)).sum(-1).to(torch.int32).view(24, 1)
    meta.tree_mask = words.cuda()
    outr = ref.paged_attention(q, kv, meta, scale)
    assert _rel_err(cu.paged_attention(q, kv, meta, scale, splits=1), outr) < 1.5e-2
    assert _rel_err(cu.paged_attention(q, kv, meta, scale, splits=3), outr) < 1.5e-2
    _sync_check(cu)


@pytest.mark.parametrize("qk_norm", [False, True])
def test_rope_kv_write(cu, qk_norm):
    hq, hkv, d, page = 8, 2, 128, 64
    q_lens, past = [5, 1, 70], [0, 130, 60]
    g = torch.Generator(device="cuda").manual_seed(2)
    t = sum(q_lens)
    n = len(q_lens)
    table = torch.arange(n * 4, dtype=torch.int32).view(n, 4)
    meta = build_step_meta(q_lens, past, table, page, device="cuda")
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda", generator=g).bfloat16()
    cs = ref.rope_cos_sin(512, d, 1e6, device="cuda")
    qw = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).bfloat16() if qk_norm else None
    kw = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).bfloat16() if qk_norm else None
    kv1 = torch.zeros(n * 4, 2, hkv, page, d, device="cuda", dtype=torch.bfloat16)
    kv2 = kv1.clone()
    q1 = cu.rope_kv_write(qkv, kv1, meta, cs, hq, hkv, d, qw, kw, 1e-6)
    q2 = ref.rope_kv_write(qkv, kv2, meta, cs, hq, hkv, d, qw, kw, 1e-6)
    assert _rel_err(q1, q2) < 6e-3
    assert _rel_err(kv1, kv2) < 6e-3
    assert torch.equal(kv1 == 0, kv2 == 0)
    _sync_check(cu)


@pytest.mark.parametrize("qk_norm,hq,hkv", [(True, 8, 2), (False, 4, 1), (True, 5, 1)])
def test_rope_kv_write_prefill_form(cu, qk_norm, hq, hkv):
    """Enough tokens for the one-warp-per-token kernel (two heads per warp pass; an odd head count leaves half a warp idle)."""
    d, page = 128, 64
    q_lens, past = [700, 400], [64, 0]
    g = torch.Generator(device="cuda").manual_seed(7)
    t, n = sum(q_lens), 2
    table = torch.arange(n * 12, dtype=torch.int32).view(n, 12)
    table[1, 5] = -1                                                    # an unreserved page is skipped, not written
    meta = build_step_meta(q_lens, past, table, page, device="cuda")
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda", generator=g).half()
    cs = ref.rope_cos_sin(1024, d, 1e4, device="cuda")
    qw = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).half() if qk_norm else None
    kw = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).half() if qk_norm else None
    kv1 = torch.zeros(n * 12, 2, hkv, page, d, device="cuda", dtype=torch.float16)
    kv2 = kv1.clone()
    q1 = cu.rope_kv_write(qkv, kv1, meta, cs, hq, hkv, d, qw, kw, 1e-6)
    table2 = table.clone()
    table2[1, 5] = 23                                                   # the reference writes there; compare everything else
    meta2 = build_step_meta(q_lens, past, table2, page, device="cuda")
    q2 = ref.rope_kv_write(qkv, kv2, meta2, cs, hq, hkv, d, qw, kw, 1e-6)
    assert _rel_err(q1, q2) < 3e-3
    keep = [i for i in range(n * 12) if i != 23]
    assert _rel_err(kv1[keep], kv2[keep]) < 3e-3 and torch.equal(kv1[keep] == 0, kv2[keep] == 0)
    _sync_check(cu)


NVFP4_SHAPES = [(256, 512, 512), (1024, 6144, 4096), (300, 1000, 768), (1, 4096, 4096), (8, 6144, 4096),
                (64, 4096, 12288), (33, 1024, 512), (128, 2048, 2048), (4096, 4096, 4096)]


@pytest.mark.parametrize("m,n,k", NVFP4_SHAPES)
def test_gemm_nvfp4(cu, m, n, k):
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    x = (torch.randn(m, k, device="cuda", generator=g)).half()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05)
    wq, wsf, wgs = ref.nvfp4_quantize(w)
    gs_x = (x.float().abs().amax() / (6 * 448)).reshape(1)
    # kernel path
    xq, xsf = cu.nvfp4_quantize(x, gs_x)
    w_atoms = cu.nvfp4_swizzle_scales(wsf)
    alpha = (wgs * gs_x).expand(n).contiguous()
    y = cu.gemm_nvfp4(xq, xsf, wq, w_atoms, alpha, torch.float16)
    torch.cuda.synchronize()
    # oracle: the same quantised operands, dequantised in fp32
    xr_q, xr_sf, _ = ref.nvfp4_quantize(x, gs_x.reshape(()))
    xd = ref.nvfp4_dequantize(xr_q, xr_sf, gs_x.reshape(()))
    wd = ref.nvfp4_dequantize(wq, wsf, wgs)
    yr = xd @ wd.t()
    # the quantiser itself: packed codes agree except at rounding ties of the reciprocal
    agree = (xq == xr_q).float().mean().item()
    assert agree > 0.97, agree
    assert _rel_err(y, yr) < 2e-2, _rel_err(y, yr)
    # and the GEMM proper, fed the oracle's own operands through the atom layout
    y2 = cu.gemm_nvfp4(xr_q, cu.nvfp4_swizzle_scales(xr_sf), wq, w_atoms, alpha, torch.float16)
    assert _rel_err(y2, yr) < 3e-3, _rel_err(y2, yr)
    _sync_check(cu)


@pytest.mark.parametrize("m,n,k", [(256, 512, 512), (1024, 6144, 4096), (300, 1000, 768), (4096, 4096, 4096), (512, 384, 1024),
                                   (130, 256, 256), (777, 2048, 12288)])
def test_gemm_nvfp4_wide_tiles_match_the_128_wide_kernel(cu, m, n, k):
    """The three prefill-size kernels — 128 x 128 tiles, 128 x 256 single CTA, 256 x 256 CTA pair (cta_group::2) — on the same
    operands: each against the fp32 oracle, and the wide ones against the 128-wide result (same products, same K order)."""
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).half()
    w = torch.randn(n, k, device="cuda", generator=g) * 0.05
    wq, wsf, wgs = ref.nvfp4_quantize(w)
    gs_x = (x.float().abs().amax() / (6 * 448)).reshape(1)
    xq, xsf = cu.nvfp4_quantize(x, gs_x)
    w_atoms = cu.nvfp4_swizzle_scales(wsf)
    alpha = (wgs * gs_x).expand(n).contiguous()
    bias = torch.randn(n, device="cuda", generator=g).half()
    resid = torch.randn(m, n, device="cuda", generator=g).half()
    xd = ref.nvfp4_dequantize(*ref.nvfp4_quantize(x, gs_x.reshape(()))[:2], gs_x.reshape(()))
    yr = xd @ ref.nvfp4_dequantize(wq, wsf, wgs).t()
    L = cu.lib()
    old = L.telb_set_nvfp4_wide_mode(0)
    try:
        outs = {}
        for mode in (0, 1, 2):
            L.telb_set_nvfp4_wide_mode(mode)
            outs[mode] = cu.gemm_nvfp4(xq, xsf, wq, w_atoms, alpha, torch.float16, mode=1)
            outs[(mode, "epi")] = cu.gemm_nvfp4(xq, xsf, wq, w_atoms, alpha, torch.float16, bias=bias, residual=resid, mode=1)
            torch.cuda.synchronize()
            cu.Workspace.get(torch.device("cuda", 0)).check_status()
    finally:
        L.telb_set_nvfp4_wide_mode(old)
    for mode in (0, 1, 2):
        assert _rel_err(outs[mode], yr) < 2e-2, (mode, _rel_err(outs[mode], yr))
        assert _rel_err(outs[(mode, "epi")], yr + bias.float() + resid.float()) < 2e-2
    for mode in (1, 2):
        assert _rel_err(outs[mode], outs[0]) < 1e-3, (mode, _rel_err(outs[mode], outs[0]))
        assert _rel_err(outs[(mode, "epi")], outs[(0, "epi")]) < 1e-3


@pytest.mark.parametrize("m,n,k,ranks", [(1, 4096, 4096, 0), (1, 512, 1024, 1), (8, 6144, 4096, 3), (16, 4096, 12288, 8),
                                         (33, 1000, 512, 2), (64, 24576, 4096, 0), (100, 4096, 4096, 5), (128, 2048, 2048, 4),
                                         (7, 151936, 4096, 0), (64, 4096, 4096, 8), (100, 1004, 512, 1), (9, 1002, 512, 1)])
def test_gemm_skinny_bf16(cu, m, n, k, ranks):
    g = torch.Generator(device="cuda").manual_seed(m + n)
    x = (torch.randn(m, k, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    b = torch.randn(n, device="cuda", generator=g).bfloat16()
    a = torch.rand(n, device="cuda", generator=g) + 0.5
    r = torch.randn(m, n, device="cuda", generator=g).bfloat16()
    y = cu.gemm_skinny(x, w, alpha=a, bias=b, residual=r, ranks=ranks)
    yr = (x.float() @ w.float().t()) * a + b.float() + r.float()
    assert _rel_err(y, yr) < 6e-3, _rel_err(y, yr)
    assert _rel_err(cu.gemm_skinny(x, w, ranks=ranks), x.float() @ w.float().t()) < 6e-3
    _sync_check(cu)


@pytest.mark.parametrize("m,n,k,ranks", [(1, 4096, 4096, 0), (8, 6144, 4096, 2), (64, 4096, 12288, 8), (33, 1024, 512, 0),
                                         (128, 2048, 2048, 4), (64, 24576, 4096, 0), (16, 2048, 768, 3)])
def test_gemm_skinny_nvfp4(cu, m, n, k, ranks):
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).half()
    w = torch.randn(n, k, device="cuda", generator=g) * 0.05
    wq, wsf, wgs = ref.nvfp4_quantize(w)
    gs_x = (x.float().abs().amax() / (6 * 448)).reshape(())
    xq, xsf, _ = ref.nvfp4_quantize(x, gs_x)
    yr = ref.nvfp4_dequantize(xq, xsf, gs_x) @ ref.nvfp4_dequantize(wq, wsf, wgs).t()
    alpha = (wgs * gs_x).expand(n).contiguous()
    y = cu.gemm_skinny(xq, wq, x_sf=cu.nvfp4_swizzle_scales(xsf), w_sf=cu.nvfp4_swizzle_scales(wsf), alpha=alpha,
                       out_dtype=torch.float16, ranks=ranks)
    assert _rel_err(y, yr) < 3e-3, _rel_err(y, yr)
    _sync_check(cu)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k,group,ranks", [(1, 4096, 4096, 128, 0), (8, 6144, 4096, 128, 3), (64, 4096, 12288, 128, 0), (100, 1000, 512, 64, 1),
                                               (33, 2048, 2048, 128, 8), (300, 1024, 1024, 128, 0), (16, 24576, 4096, 128, 0)])
def test_gemm_int4_awq_in_kernel(cu, m, n, k, group, ranks, dtype):
    """W4A16 on ModelOpt-prepacked INT4 weights: decode sizes expand the 4-bit tiles inside the GEMM kernel (every cluster
    size), larger steps go through the expand kernel + dense GEMM; both against the fp32 statement (q - 8) * scale."""
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).to(dtype)
    wq = torch.randint(0, 256, (n // 2, k), device="cuda", generator=g, dtype=torch.uint8)
    scales = (torch.rand(n, k // group, device="cuda", generator=g) * 0.02 + 0.005).to(dtype)
    bias = torch.randn(n, device="cuda", generator=g).to(dtype)
    wd = ref.int4_awq_dequantize(wq, scales, None, group)
    want = x.float() @ wd.t() + bias.float()
    got = cu.gemm_int4_awq(x, wq, scales, group, bias=bias, ranks=ranks)
    torch.cuda.synchronize()
    assert got.shape == (m, n)
    assert _rel_err(got, want) < 6e-3, _rel_err(got, want)
    _sync_check(cu)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k,group", [(1, 6144, 4096, 128), (2, 4096, 12288, 128), (3, 1000, 512, 64), (4, 24576, 4096, 128), (1, 64, 128, 64)])
def test_gemv_int4_awq_few_rows(cu, m, n, k, group, dtype, monkeypatch):
    """One to four rows take the CUDA-core GEMV (exact code expansion, fp32 sums): against the fp32 statement, with bias and
    residual, and against the tensor-core path with the GEMV switched off."""
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).to(dtype)
    wq = torch.randint(0, 256, (n // 2, k), device="cuda", generator=g, dtype=torch.uint8)
    scales = (torch.rand(n, k // group, device="cuda", generator=g) * 0.02 + 0.005).to(dtype)
    bias = torch.randn(n, device="cuda", generator=g).to(dtype)
    res = torch.randn(m, n, device="cuda", generator=g).to(dtype)
    wd = ref.int4_awq_dequantize(wq, scales, None, group)
    want = x.float() @ wd.t() + bias.float() + res.float()
    assert cu.INT4_GEMV_MAX_ROWS == 4
    got = cu.gemm_int4_awq(x, wq, scales, group, bias=bias, residual=res)
    torch.cuda.synchronize()
    assert got.shape == (m, n) and _rel_err(got, want) < 4e-3, _rel_err(got, want)
    monkeypatch.setattr(cu, "INT4_GEMV_MAX_ROWS", 0)
    if k % 64 == 0 and group % 64 == 0:
        other = cu.gemm_int4_awq(x, wq, scales, group, bias=bias, residual=res)
        assert _rel_err(got, other.float()) < 6e-3
    _sync_check(cu)


def test_skinny_chain_in_cuda_graph(cu):
    """Back-to-back decode GEMMs launched with programmatic dependent launch, captured and replayed."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(8, 1024, device="cuda", generator=g) * 0.5).bfloat16()
    w1 = (torch.randn(2048, 1024, device="cuda", generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(1024, 2048, device="cuda", generator=g) * 0.05).bfloat16()
    yr = ((x.float() @ w1.float().t()).bfloat16().float() @ w2.float().t())
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        y = cu.gemm(cu.gemm(x, w1), w2)
    torch.cuda.current_stream().wait_stream(s)
    assert _rel_err(y, yr) < 1e-2
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y2 = cu.gemm(cu.gemm(x, w1), w2)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert _rel_err(y2, yr) < 1e-2
    _sync_check(cu)


def test_fused_norm_and_swiglu_quant(cu):
    g = torch.Generator(device="cuda").manual_seed(11)
    for rows, hidden in [(5, 4096), (130, 2048), (64, 12288), (3, 768)]:
        x = torch.randn(rows, hidden, device="cuda", generator=g).half()
        r = torch.randn(rows, hidden, device="cuda", generator=g).half()
        w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).half()
        gs = torch.tensor([0.01], device="cuda")
        qa, res = cu.rmsnorm_quant(x, r, w, 1e-6, gs)
        y_ref, res_ref = ref.add_rmsnorm(x, r, w, 1e-6)
        assert torch.equal(res, res_ref)
        xq2, sf2 = cu.nvfp4_quantize(cu.add_rmsnorm(x, r, w, 1e-6)[0], gs)
        assert (qa.xq == xq2).float().mean().item() > 0.995
        # dequantised result tracks the 16-bit normalised activations
        p_ref, sf_ref, _ = ref.nvfp4_quantize(y_ref, gs.reshape(()))
        assert (qa.xq == p_ref).float().mean().item() > 0.97
        qa1, res1 = cu.rmsnorm_quant(x, None, w, 1e-6, gs)
        assert res1 is x
        assert (qa1.xq == cu.nvfp4_quantize(cu.rmsnorm(x, w, 1e-6), gs)[0]).float().mean().item() > 0.995
    gu = torch.randn(70, 2 * 1536, device="cuda", generator=g).half()
    gs = torch.tensor([0.02], device="cuda")
    qa = cu.swiglu_quant(gu, gs)
    xq2, sf2 = cu.nvfp4_quantize(cu.swiglu(gu), gs)
    assert (qa.xq == xq2).float().mean().item() > 0.995
    # end to end through a GEMM
    w = torch.randn(512, 1536, device="cuda", generator=g) * 0.05
    wq, wsf, wgs = ref.nvfp4_quantize(w)
    alpha = (wgs * gs).expand(512).contiguous()
    y1 = cu.gemm_nvfp4(qa.xq, qa.sf, wq, cu.nvfp4_swizzle_scales(wsf), alpha, torch.float16)
    y2 = cu.gemm_nvfp4(xq2, sf2, wq, cu.nvfp4_swizzle_scales(wsf), alpha, torch.float16)
    assert _rel_err(y1, y2) < 5e-3
    _sync_check(cu)


def test_gemm_nvfp4_swiglu_epilogue_matches_unfused_chain():
    """Gate/up GEMM with SwiGLU + NVFP4 quantisation in the epilogue == GEMM → swiglu_quant, bit for bit."""
    from tensorrt_edge_llm_b200.ops import cuda as cu
    torch.manual_seed(0)
    m, k, inter = 300, 512, 384
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(m, k, device="cuda", generator=g).half()
    wq = torch.randint(0, 256, (2 * inter, k // 2), device="cuda", generator=g, dtype=torch.uint8)
    wsf = torch.randint(48, 58, (2 * inter, k // 16), device="cuda", generator=g, dtype=torch.uint8)
    alpha = (torch.rand(2 * inter, device="cuda", generator=g) * 0.02 + 0.01)
    gs_in = torch.full((1,), 1.0 / 448, device="cuda")
    gs_out = torch.full((1,), 0.004, device="cuda")
    xq, xsf = cu.nvfp4_quantize(x, gs_in)
    acts = cu.QuantActs(xq, xsf, (m, k), torch.float16)
    # unfused: plain [gate | up] weights
    gu = cu.gemm_nvfp4(xq, xsf, wq, cu.nvfp4_swizzle_scales(wsf), alpha, torch.float16, mode=1)
    want = cu.swiglu_quant(gu, gs_out)
    # fused: rows interleaved in blocks of 64
    blk = torch.arange(inter, device="cuda").view(inter // 64, 64)
    perm = torch.stack([blk, blk + inter], 1).reshape(-1)
    w_il, sf_il, a_il = wq[perm].contiguous(), wsf[perm].contiguous(), alpha[perm].contiguous()
    got = cu.gemm_nvfp4_swiglu(acts, w_il, cu.nvfp4_swizzle_scales(sf_il), a_il, gs_out)
    torch.cuda.synchronize()
    assert torch.equal(got.xq, want.xq)
    assert torch.equal(got.sf[: want.sf.numel()].view(torch.uint8), want.sf.view(torch.uint8)[: got.sf.numel()])
    # the decode-size path reads the interleaved GEMM output
    gu_il = cu.gemm_nvfp4(xq, xsf, w_il, cu.nvfp4_swizzle_scales(sf_il), a_il, torch.float16, mode=1)
    small = cu.swiglu_quant(gu_il, gs_out, interleaved=True)
    assert torch.equal(small.xq, want.xq)
    cu.Workspace.get(torch.device("cuda", 0)).check_status()


@pytest.mark.parametrize("m,k,inter", [(1, 512, 384), (8, 4096, 1536), (33, 1024, 768), (64, 4096, 3072), (64, 512, 128)])
def test_gemm_skinny_swiglu_epilogue_matches_unfused_chain(m, k, inter):
    """Decode-size gate/up GEMM with SwiGLU + NVFP4 quantisation in its epilogue == skinny GEMM → swiglu_quant, bit for bit
    (single CTA per tile and every cluster size the chooser picks for these shapes)."""
    from tensorrt_edge_llm_b200.ops import cuda as cu
    g = torch.Generator(device="cuda").manual_seed(m + k)
    x = torch.randn(m, k, device="cuda", generator=g).half()
    wq = torch.randint(0, 256, (2 * inter, k // 2), device="cuda", generator=g, dtype=torch.uint8)
    wsf = torch.randint(48, 58, (2 * inter, k // 16), device="cuda", generator=g, dtype=torch.uint8)
    alpha = (torch.rand(2 * inter, device="cuda", generator=g) * 0.02 + 0.01)
    gs_in = torch.full((1,), 1.0 / 448, device="cuda")
    gs_out = torch.full((1,), 0.004, device="cuda")
    xq, xsf = cu.nvfp4_quantize(x, gs_in)
    acts = cu.QuantActs(xq, xsf, (m, k), torch.float16)
    atoms = cu.nvfp4_swizzle_scales(wsf)
    gu = cu.gemm_nvfp4(xq, xsf, wq, atoms, alpha, torch.float16)                 # decode-size kernel, interleaved rows
    want = cu.swiglu_quant(gu, gs_out, interleaved=True)
    got = cu.gemm_skinny_swiglu(acts, wq, atoms, alpha, gs_out)
    torch.cuda.synchronize()
    assert torch.equal(got.xq, want.xq)
    idx = _sf_rows_index(m, inter)                         # rows past m inside the 128-row atom hold anything
    assert torch.equal(got.sf.view(torch.uint8)[idx], want.sf.view(torch.uint8)[idx])
    cu.Workspace.get(torch.device("cuda", 0)).check_status()


def test_mlp_with_fused_swiglu_matches_unfused(monkeypatch):
    """A whole NVFP4 MLP: prefill rows through the fused epilogue, decode rows through the interleaved kernel, both equal
    to the layer built with the fusion switched off."""
    from tensorrt_edge_llm_b200.config import QUANT_NVFP4, QuantConfig, tiny_llama_config
    from tensorrt_edge_llm_b200.models.default import MLP
    from tensorrt_edge_llm_b200 import ops
    cfg = tiny_llama_config(hidden_size=512, intermediate_size=768, dtype="float16")
    cfg.quant = QuantConfig(quant_type=QUANT_NVFP4, group_size=16)

    def build():
        torch.manual_seed(3)
        mlp = MLP(cfg, "model.layers.0.mlp")
        gen = torch.Generator().manual_seed(5)
        mlp.gate_up_proj.quantize_from([torch.randn(768, 512, generator=gen) * 0.05, torch.randn(768, 512, generator=gen) * 0.05])
        mlp.down_proj.quantize_from([torch.randn(512, 768, generator=gen) * 0.05])
        return mlp.cuda()
    fused = build()
    monkeypatch.setenv("TELB_DISABLE_SWIGLU_FUSION", "1")
    plain = build()
    assert fused.gate_up_proj.want_interleave and not plain.gate_up_proj.want_interleave
    w = torch.ones(512, device="cuda", dtype=torch.float16)
    for rows in (400, 16):
        x = torch.randn(rows, 512, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rows)).half()
        qa = ops.rmsnorm_maybe_quant(x, w, 1e-6, fused.gate_up_proj.fused_input_scale())
        qb = ops.rmsnorm_maybe_quant(x, w, 1e-6, plain.gate_up_proj.fused_input_scale())
        assert torch.equal(fused(qa), plain(qb))
    assert fused.gate_up_proj.gate_up_interleaved and not plain.gate_up_proj.gate_up_interleaved
    assert torch.equal(fused.gate_up_proj.dequantized_weight(), plain.gate_up_proj.dequantized_weight())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,vocab,k", [(1, 100, 0), (5, 4099, 5), (64, 151936, 20), (3, 33, 32)])
def test_token_logprobs_kernel(dtype, rows, vocab, k):
    """Chosen-token and top-k log-probabilities against log_softmax + a stable sort of the same (rounded) logits."""
    from tensorrt_edge_llm_b200.ops import cuda as cu
    g = torch.Generator().manual_seed(vocab + k)
    logits = (torch.randn(rows, vocab, generator=g) * 4).to(dtype)
    logits[0, 7] = logits[0, 3] = logits.float().max() + 1       # a tie at the top: the lower id first
    if vocab > 50:
        logits[-1, 40:50] = float("-inf")                        # masked tokens (guided decoding)
    tokens = torch.randint(0, vocab, (rows,), generator=g)
    want = ref.token_logprobs(logits, tokens, k)
    got = cu.token_logprobs(logits.cuda(), tokens.cuda(), k)
    assert torch.allclose(got[0].cpu(), want[0], atol=2e-3)
    if k:
        assert torch.equal(got[1].cpu(), want[1]) and torch.allclose(got[2].cpu(), want[2], atol=2e-3)
        assert got[1][0, :2].tolist() == [3, 7]
    # a strided view (the last rows of a wider buffer) reads the right rows
    wide = torch.zeros(rows, vocab + 8, dtype=dtype).cuda()
    wide[:, :vocab] = logits.cuda()
    again = cu.token_logprobs(wide[:, :vocab], tokens.cuda(), k)
    assert torch.allclose(again[0], got[0]) and torch.equal(again[1], got[1])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fmt", ["fp8", "nvfp4"])
def test_quantized_embedding_gather_kernel(fmt, dtype):
    """Gather + expand of FP8 / NVFP4 embedding rows in one kernel against the torch expansion of the same stored table."""
    from tensorrt_edge_llm_b200.models.embedding import QuantizedEmbedding
    g = torch.Generator().manual_seed(3)
    table = (torch.randn(1000, 256, generator=g) * 0.05).to(dtype)
    emb = QuantizedEmbedding.from_dense(table, fmt)
    ids = torch.randint(0, 1000, (3, 17), generator=g)
    want = emb(ids)                                           # CPU: torch ops
    got = emb.cuda()(ids.cuda())
    assert got.shape == (3, 17, 256) and got.dtype == dtype
    assert torch.allclose(got.float().cpu(), want.float(), atol=1e-3, rtol=1e-2)
    assert torch.allclose(got.float().cpu(), table[ids].float(), atol=0.03 if fmt == "nvfp4" else 0.02)
    out_of_range = emb.cuda()(torch.tensor([-5, 5000]).cuda())      # clamped like the dense gather
    assert torch.equal(out_of_range[0], emb.cuda()(torch.tensor([0]).cuda())[0]) and torch.equal(out_of_range[1], emb.cuda()(torch.tensor([999]).cuda())[0])


@pytest.mark.parametrize("d,tokens", [(128, 5), (128, 1500), (64, 33), (256, 9)])
def test_rope_q_only_writes_no_cache(d, tokens):
    """Queries of a KV-shared layer: per-head RMSNorm + RoPE through the RoPE / KV-write kernels with zero KV heads."""
    from tensorrt_edge_llm_b200 import ops
    g = torch.Generator().manual_seed(d + tokens)
    hq = 4
    q = torch.randn(tokens, hq * d, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16)
    cs = ref.rope_cos_sin(4096, d, 1e4, None)
    pages = (tokens + 63) // 64
    meta = build_step_meta([tokens], [7], torch.arange(pages + 1, dtype=torch.int32)[None], 64)
    kv = torch.full((pages + 1, 2, 2, 64, d), 3.0, dtype=torch.bfloat16)
    want = ref.rope_q(q.float(), meta, cs, hq, d, w.float(), 1e-6)
    kv_gpu = kv.cuda()
    got = ops.rope_q(q.cuda(), kv_gpu, meta.to("cuda"), cs.cuda(), hq, d, w.cuda(), 1e-6)
    assert got.shape == (tokens, hq, d) and _rel_err(got.float().cpu(), want) < 2e-2
    assert torch.equal(kv_gpu.cpu(), kv)                      # nothing was stored


def test_kv_shared_layers_gpu_matches_cpu():
    from tensorrt_edge_llm_b200 import AutoModel
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
    from tensorrt_edge_llm_b200.runtime.runner import ModelRunner
    cfg = tiny_llama_config(num_hidden_layers=4, hidden_size=512, intermediate_size=1024, num_attention_heads=8, num_key_value_heads=2,
                            head_dim=128, vocab_size=1000, dtype="bfloat16")
    cfg.num_kv_shared_layers = 2
    model = AutoModel.from_config(cfg, random_init=0)
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    seq = torch.randint(0, 1000, (70,), generator=torch.Generator().manual_seed(1)).tolist()

    def run(device):
        m = AutoModel.from_config(cfg)
        m.load_state_dict(sd)
        m = m.to(device)
        r = ModelRunner(m, KVCacheManager(cfg, num_pages=8, page_size=64, max_seats=2, max_pages_per_seq=4, device=device))
        r.use_cuda_graphs = False
        return r.prefill([0], [seq[:-2]]).float().cpu(), r.step([0], [[seq[-2]]]).float().cpu(), r.step([0], [[seq[-1]]]).float().cpu()

    for x, y in zip(run(torch.device("cuda", 0)), run(torch.device("cpu"))):
        assert _rel_err(x, y) < 5e-2


@pytest.mark.parametrize("scaling", [None, {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 8192},
                                     {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 4096}])
def test_rope_table_and_mrope_rows_kernels(scaling):
    """RoPE table built on the device (fp64 angles) against the host table, at positions where fp32 angles would have lost
    their fraction; multimodal rows gathered by (t, h, w) positions against the torch gather."""
    from tensorrt_edge_llm_b200 import ops
    want = ref.rope_cos_sin(40000, 128, 1e6, scaling)
    got = ops.rope_cos_sin(40000, 128, 1e6, scaling, device="cuda")
    assert got.shape == want.shape and got.dtype == torch.float32
    assert float((got.cpu() - want).abs().max()) < 2e-6
    g = torch.Generator().manual_seed(0)
    pos3 = torch.randint(0, 40000, (3, 77), generator=g, dtype=torch.int32)
    sections = [16, 24, 24]
    rows = ops.mrope_rows(got, pos3.cuda(), sections)
    assert torch.equal(rows.cpu(), ref.mrope_rows(got.cpu(), pos3, sections))
    with pytest.raises(ValueError):
        ops.mrope_rows(got, pos3.cuda(), [16, 16, 16])
