"""FP8 (E4M3) KV-cache storage on the host formulation: half the bytes per token, outputs that track the unquantised cache."""
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import QuantConfig, tiny_llama_config
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def _run(model, cfg, prompts, feed, kv_dtype):
    kv = KVCacheManager(cfg, num_pages=16, page_size=64, max_seats=2, max_pages_per_seq=4, kv_dtype=kv_dtype)
    r = ModelRunner(model, kv)
    out = [r.prefill([0, 1], prompts)]
    for toks in feed:
        out.append(r.step([0, 1], [[t] for t in toks]))
    return torch.stack(out), kv


def test_fp8_kv_cache_tracks_the_unquantised_cache():
    cfg = tiny_llama_config(num_hidden_layers=2, vocab_size=512, dtype="float32", head_dim=64, num_attention_heads=4, num_key_value_heads=2,
                            hidden_size=256)
    model = AutoModel.from_config(cfg, random_init=0)
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(0, cfg.vocab_size, (2, 90), generator=g).tolist()           # crosses a page boundary
    feed = torch.randint(0, cfg.vocab_size, (6, 2), generator=g).tolist()               # teacher forcing: same tokens for both runs
    full, kv16 = _run(model, cfg, prompts, feed, None)
    fp8, kv8 = _run(model, cfg, prompts, feed, "fp8")
    assert kv8.pool.dtype == torch.float8_e4m3fn and kv8.bytes_per_token * 4 == kv16.bytes_per_token      # fp32 reference pool here
    cos = torch.nn.functional.cosine_similarity(full.flatten(1), fp8.flatten(1), dim=1)
    assert float(cos.min()) > 0.999, cos
    # per-layer scales widen the range: values beyond 448 survive with a calibrated scale
    for layer in model.model.layers:
        layer.self_attn.kv_scales.copy_(torch.tensor([0.5, 2.0]))
    scaled, _ = _run(model, cfg, prompts, feed, "fp8")
    assert float(torch.nn.functional.cosine_similarity(full.flatten(1), scaled.flatten(1), dim=1).min()) > 0.998
    # the checkpoint's quantisation config selects FP8 pages by itself
    cfg.quant = QuantConfig(kv_cache_quant="fp8")
    assert KVCacheManager(cfg, num_pages=4, page_size=64, max_seats=1, max_pages_per_seq=2).kv_fp8
    assert not KVCacheManager(cfg, num_pages=4, page_size=64, max_seats=1, max_pages_per_seq=2, kv_dtype="model").kv_fp8
