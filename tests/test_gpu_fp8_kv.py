"""FP8 (E4M3) KV-cache storage on the GPU: the load / store kernels against the host formulation, and a model whose outputs
track the 16-bit cache through prefill, eager decode steps and graph-replayed decode."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.ops import build_step_meta
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_kv_fp8_load_and_store_kernels(dtype):
    from tensorrt_edge_llm_b200.ops import cuda as cu
    g = torch.Generator().manual_seed(2)
    pages, hkv, psz, d = 12, 2, 64, 128
    q_lens, pasts = [5, 1, 70], [100, 0, 64]
    table = torch.full((3, 4), -1, dtype=torch.int32)
    table[0, :2] = torch.tensor([7, 2]); table[1, :1] = torch.tensor([9]); table[2, :3] = torch.tensor([4, 0, 11])
    meta_c = build_step_meta(q_lens, pasts, table, psz)
    meta_g = meta_c.to("cuda")
    scales = torch.tensor([0.25, 3.0])
    pool = (torch.randn(pages, 2, hkv, psz, d, generator=g) * 40).to(torch.float8_e4m3fn)
    stage0 = torch.randn(pages, 2, hkv, psz, d, generator=g).to(dtype)           # stale contents that must survive where untouched
    # load
    want = stage0.clone()
    ref.kv_fp8_load(pool, want, meta_c, scales)
    got = stage0.clone().cuda()
    cu.kv_fp8_load(pool.cuda(), got, meta_g, scales.cuda())
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), want)
    # store: new rows (written 16-bit into the staging layer) land in the pool as E4M3 and are rounded in place
    new = want.clone()
    new += (torch.randn(new.shape, generator=g) * 30).to(dtype)
    pool_w, stage_w = pool.clone(), new.clone()
    ref.kv_fp8_store(pool_w, stage_w, meta_c, scales)
    pool_g, stage_g = pool.clone().cuda(), new.clone().cuda()
    cu.kv_fp8_store(pool_g, stage_g, meta_g, scales.cuda())
    torch.cuda.synchronize()
    assert torch.equal(pool_g.cpu().view(torch.uint8), pool_w.view(torch.uint8))
    assert torch.equal(stage_g.cpu(), stage_w)
    cu.Workspace.get(torch.device("cuda", 0)).check_status()


@pytest.mark.parametrize("case", [([1], [100], 32, 8, 64), ([1, 1, 1], [5, 64, 700], 32, 8, 64), ([1] * 9, [0, 1, 63, 64, 127, 128, 129, 1000, 2047], 32, 8, 64),
                                  ([2, 1, 4], [10, 300, 77], 16, 4, 64), ([1, 1], [500, 90], 16, 1, 64), ([1, 3], [150, 260], 32, 8, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_attention_reads_fp8_pages_in_place(case, dtype):
    """The decode kernel's E4M3 variant (K, V, Q and the probabilities enter the tensor cores as E4M3) against the fp32 statement
    on the dequantised operands, with and without KV splits, a sliding window and the NVFP4 output epilogue."""
    from tensorrt_edge_llm_b200.ops import cuda as cu
    q_lens, past_lens, hq, hkv, page = case
    d = 128
    g = torch.Generator().manual_seed(sum(past_lens) + hq)
    n = len(q_lens)
    max_pages = max((a + b + page - 1) // page for a, b in zip(q_lens, past_lens)) + 1
    total = n * max_pages + 2
    perm = torch.randperm(total, generator=g)
    table = torch.full((n, max_pages), -1, dtype=torch.int32)
    k = 0
    for s_ in range(n):
        need = (q_lens[s_] + past_lens[s_] + page - 1) // page
        table[s_, :need] = perm[k:k + need].to(torch.int32)
        k += need
    meta = build_step_meta(q_lens, past_lens, table, page).to("cuda")
    scales = torch.tensor([0.02, 0.05])
    kv = torch.randn(total, 2, hkv, page, d, generator=g)
    pool = (kv / scales.view(1, 2, 1, 1, 1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    kv_deq = (pool.float() * scales.view(1, 2, 1, 1, 1)).to(dtype)
    q = torch.randn(sum(q_lens), hq, d, generator=g).to(dtype)
    q8 = q.float().clamp(-448, 448).to(torch.float8_e4m3fn)
    scale = d ** -0.5
    meta_c = build_step_meta(q_lens, past_lens, table, page)
    want = ref.paged_attention(q8.float().to(dtype), kv_deq, meta_c, scale).float()
    for splits in (1, 3):
        got = cu.paged_attention_decode_fp8(q8.cuda(), pool.cuda(), meta, scale, None, scales.cuda(), dtype, splits=splits)
        torch.cuda.synchronize()
        err = (got.float().cpu() - want).norm() / want.norm()
        cos = torch.nn.functional.cosine_similarity(got.float().cpu().flatten(), want.flatten(), dim=0)
        # E4M3 probabilities carry ~3.6 % rms error per element, which the flat attention of random inputs does not average away
        assert err < 8e-2 and cos > 0.997, (splits, float(err), float(cos))
    want_w = ref.paged_attention(q8.float().to(dtype), kv_deq, meta_c, scale, sliding_window=100).float()
    got_w = cu.paged_attention_decode_fp8(q8.cuda(), pool.cuda(), meta, scale, 100, scales.cuda(), dtype)
    assert (got_w.float().cpu() - want_w).norm() / want_w.norm() < 8e-2
    # NVFP4 epilogue == the 16-bit output through the stand-alone quantiser
    gs = torch.tensor(0.004, device="cuda")
    plain = cu.paged_attention_decode_fp8(q8.cuda(), pool.cuda(), meta, scale, None, scales.cuda(), dtype, splits=1)
    xq_ref, _ = cu.nvfp4_quantize(plain.reshape(plain.shape[0], -1), gs)
    qa = cu.paged_attention_decode_fp8(q8.cuda(), pool.cuda(), meta, scale, None, scales.cuda(), dtype, out_scale=gs, splits=1)
    torch.cuda.synchronize()
    assert torch.equal(qa.xq, xq_ref)
    cu.Workspace.get(torch.device("cuda", 0)).check_status()


def test_model_with_fp8_kv_tracks_16_bit_cache_eager_and_graph():
    dev = torch.device("cuda", 0)
    cfg = tiny_llama_config(num_hidden_layers=3, vocab_size=512, dtype="bfloat16", head_dim=128, num_attention_heads=4, num_key_value_heads=2,
                            hidden_size=512)
    model = AutoModel.from_config(cfg, device=dev, random_init=0)
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(0, cfg.vocab_size, (2, 300), generator=g).tolist()
    feed = torch.randint(0, cfg.vocab_size, (5, 2), generator=g).tolist()

    def run(kv_dtype):
        kv = KVCacheManager(cfg, num_pages=24, page_size=64, max_seats=2, max_pages_per_seq=10, device=dev, kv_dtype=kv_dtype)
        r = ModelRunner(model, kv, max_num_tokens=256)          # chunked prefill: later chunks read FP8 pages of earlier ones
        out = [r.prefill([0, 1], prompts).float()]
        for toks in feed:
            out.append(r.step([0, 1], [[t] for t in toks]).float())
        first = out[-1].argmax(-1).to(torch.int32)
        toks = r.decode_greedy([0, 1], first, 12)                # captured decode steps
        return torch.stack(out).cpu(), toks.cpu(), kv

    full, toks16, kv16 = run(None)
    fp8, toks8, kv8 = run("fp8")
    assert kv8.pool.dtype == torch.float8_e4m3fn and kv8.bytes_per_token * 2 == kv16.bytes_per_token
    cos = torch.nn.functional.cosine_similarity(full.flatten(1), fp8.flatten(1), dim=1)
    assert float(cos.min()) > 0.999, cos
    assert toks8.shape == toks16.shape and (toks8 == toks16).float().mean() > 0.5      # random weights: near ties may flip a token
    # determinism: the FP8 run repeats bit for bit
    fp8b, toks8b, _ = run("fp8")
    assert torch.equal(fp8, fp8b) and torch.equal(toks8, toks8b)
