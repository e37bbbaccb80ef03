"""Hybrid decoder (Mamba2 + gated DeltaNet + attention) on CPU: the recurrent state carried across
chunked prefill and decode steps must reproduce a single full-sequence pass."""
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import GdnConfig, MambaConfig, hybrid_nemotron_config
from tensorrt_edge_llm_b200.ops import build_step_meta
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def _cfg():
    return hybrid_nemotron_config(num_hidden_layers=8, vocab_size=500, hidden_size=64, intermediate_size=128, num_attention_heads=4,
                                  num_key_value_heads=2, head_dim=16, dtype="float32", max_position_embeddings=512,
                                  mamba=MambaConfig(num_heads=4, head_dim=8, d_state=16, n_groups=2, conv_kernel=4),
                                  gdn=GdnConfig(num_k_heads=2, num_v_heads=4, head_k_dim=8, head_v_dim=8, conv_kernel=4))


def _runner(model, max_tokens=8192):
    kv = KVCacheManager(model.cfg, num_pages=32, page_size=16, max_seats=4, max_pages_per_seq=8)
    return ModelRunner(model, kv, max_num_tokens=max_tokens)


def test_layer_pattern_and_state_pools():
    cfg = _cfg()
    assert cfg.layer_types.count("attention") == 1 and cfg.layer_types.count("gdn") == 1 and cfg.layer_types.count("mamba") == 6
    model = AutoModel.from_config(cfg, random_init=0)
    r = _runner(model)
    assert r.kv.pool.shape[0] == 1 and len(r.kv.recurrent.ssm) == 6 and len(r.kv.recurrent.gdn) == 1
    assert r.kv.recurrent.bytes() > 0


def test_chunked_prefill_and_decode_match_full_pass():
    cfg = _cfg()
    model = AutoModel.from_config(cfg, random_init=0)
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (45, 70)]
    full = _runner(model)
    want = full.prefill([0, 1], seqs)                              # one pass over whole prompts
    chunked = _runner(model, max_tokens=32)                        # forces 16-token-aligned chunks
    got = chunked.prefill([0, 1], seqs)
    assert (got - want).abs().max() < 2e-4
    # prefill all but the last 3 tokens, then feed those one at a time
    step = _runner(model)
    step.prefill([0, 1], [s[:-3] for s in seqs])
    for k in range(3, 0, -1):
        logits = step.step([0, 1], [[s[-k]] for s in seqs])
    assert (logits - want).abs().max() < 2e-4
    # the second sequence alone gives the same answer (state rows are independent)
    solo = _runner(model)
    assert (solo.prefill([2], [seqs[1]])[0] - want[1]).abs().max() < 2e-4


def test_recurrent_reference_ops_are_consistent():
    g = torch.Generator().manual_seed(1)
    t, c, w = 12, 6, 4
    x = torch.randn(t, c, generator=g)
    weight, bias = torch.randn(c, w, generator=g), torch.randn(c, generator=g)
    table = torch.zeros(1, 1, dtype=torch.int32)
    st_full = torch.zeros(2, c, w - 1)
    y_full = ref.causal_conv1d(x, weight, bias, st_full, build_step_meta([t], [0], table, 16), True)
    st = torch.zeros(2, c, w - 1)
    y1 = ref.causal_conv1d(x[:5], weight, bias, st, build_step_meta([5], [0], table, 16), True)
    y2 = ref.causal_conv1d(x[5:], weight, bias, st, build_step_meta([7], [5], table, 16), True)
    assert torch.allclose(torch.cat([y1, y2]), y_full, atol=1e-6) and torch.allclose(st, st_full)
    # gated delta rule: step-by-step equals one call
    hk, hv, kd, vd = 2, 4, 8, 8
    q, k = torch.randn(t, hk, kd, generator=g), torch.randn(t, hk, kd, generator=g)
    v, a, b = torch.randn(t, hv, vd, generator=g), torch.randn(t, hv, generator=g), torch.randn(t, hv, generator=g)
    A_log, dtb = torch.randn(hv, generator=g), torch.randn(hv, generator=g)
    s1 = torch.zeros(1, hv, kd, vd)
    o_full = ref.gated_delta_rule(q, k, v, a, b, A_log, dtb, s1, build_step_meta([t], [0], table, 16))
    s2 = torch.zeros(1, hv, kd, vd)
    outs = [ref.gated_delta_rule(q[i:i + 1], k[i:i + 1], v[i:i + 1], a[i:i + 1], b[i:i + 1], A_log, dtb, s2,
                                 build_step_meta([1], [i], table, 16)) for i in range(t)]
    assert torch.allclose(torch.cat(outs), o_full, atol=1e-5) and torch.allclose(s1, s2, atol=1e-5)


def test_prefix_reuse_restores_recurrent_snapshots():
    """In-flight batching with the prefix cache on a hybrid model: shared pages come with the recurrent rows saved at
    the same page boundary, so a repeated prompt (and a prompt sharing a prefix) gives the tokens of a cold run."""
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams
    cfg = _cfg()
    g = torch.Generator().manual_seed(11)
    base = torch.randint(0, 500, (75,), generator=g).tolist()
    other = base[:48] + torch.randint(0, 500, (20,), generator=g).tolist()          # shares three 16-token pages
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    kw = dict(device="cpu", max_batch_size=2, max_input_len=128, max_kv_cache_capacity=160, page_size=16, enable_in_flight_batching=True,
              scheduling={"mode": "mixed", "max_num_tokens": 64, "max_chunk_tokens": 32})
    cold = LLM(cfg, **kw)
    want_base, want_other = (o.token_ids for o in cold.generate([base, other], sp))
    cold.close()
    warm = LLM(cfg, enable_prefix_cache=True, **kw)
    assert warm.generate([base], sp)[0].token_ids == want_base
    reused0 = warm.engine.metrics().prefix_reused_tokens
    assert warm.generate([base], sp)[0].token_ids == want_base                     # 64 of 75 tokens reused with their state
    assert warm.engine.metrics().prefix_reused_tokens - reused0 == 64
    # 48 tokens are shared, but snapshots exist where prefill chunks ended (32, 64): the longest usable prefix is 32
    assert warm.generate([other], sp)[0].token_ids == want_other
    assert warm.engine.metrics().prefix_reused_tokens - reused0 == 64 + 32
    warm.close()
