"""KV-shared layers: the last layers of a decoder project queries only and attend over an earlier layer's cache."""
import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def test_donor_rule():
    cfg = tiny_llama_config(num_hidden_layers=6, dtype="float32")
    assert [cfg.kv_donor(i) for i in range(6)] == [-1] * 6
    cfg.num_kv_shared_layers = 2
    assert [cfg.kv_donor(i) for i in range(6)] == [-1, -1, -1, -1, 3, 3]
    # with alternating attention types a shared layer takes the last earlier layer of its own type
    cfg.layer_windows = [8, 0, 8, 0, 8, 0]
    assert [cfg.kv_donor(i) for i in range(6)] == [-1, -1, -1, -1, 2, 3]
    cfg.kv_donor_layers = [-1, 0, -1, 2, 2, 0]
    assert [cfg.kv_donor(i) for i in range(6)] == [-1, 0, -1, 2, 2, 0]
    cfg.kv_donor_layers = [-1, 3, -1, -1, -1, -1]
    with pytest.raises(ValueError):
        cfg.kv_donor(1)
    cfg.kv_donor_layers, cfg.num_kv_shared_layers = [], 6
    with pytest.raises(ValueError):
        cfg.kv_donor(0)


def test_shared_layers_match_a_dense_restatement_and_decode_consistently():
    cfg = tiny_llama_config(num_hidden_layers=4, dtype="float32")
    cfg.num_kv_shared_layers = 2
    model = AutoModel.from_config(cfg, random_init=5)
    shared = model.model.layers[3].self_attn
    assert shared.kv_donor == 1 and model.model.layers[2].self_attn.kv_donor == 1 and model.model.layers[1].self_attn.kv_donor == -1
    # a shared layer carries a query projection only
    assert tuple(shared.qkv_proj.weight.shape) == (cfg.q_size, cfg.hidden_size)
    g = torch.Generator().manual_seed(0)
    seq = torch.randint(0, cfg.vocab_size, (21,), generator=g).tolist()

    # dense restatement: plain causal attention per layer, layers 2 and 3 reuse layer 1's rotated keys and its values
    def dense(ids):
        t = len(ids)
        h = model.model.embed_tokens.weight[torch.tensor(ids)]
        cs = model.cos_sin("cpu")
        pos = torch.arange(t)
        kept = {}
        for i, layer in enumerate(model.model.layers):
            a = layer.self_attn
            x = ref.rmsnorm(h, layer.input_layernorm.weight, layer.input_layernorm.eps)
            proj = x @ a.qkv_proj.weight.t()
            if a.kv_donor < 0:
                q, k, v = proj.split([cfg.q_size, cfg.kv_size, cfg.kv_size], -1)
                k = ref.apply_rope(k.reshape(t, cfg.num_key_value_heads, cfg.head_dim), pos, cs)
                v = v.reshape(t, cfg.num_key_value_heads, cfg.head_dim)
                kept[i] = (k, v)
            else:
                q, (k, v) = proj, kept[a.kv_donor]
            q = ref.apply_rope(q.reshape(t, cfg.num_attention_heads, cfg.head_dim), pos, cs)
            rep = cfg.num_attention_heads // cfg.num_key_value_heads
            kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
            sc = torch.einsum("qhd,khd->hqk", q, kk) * cfg.head_dim ** -0.5
            sc = sc.masked_fill(torch.triu(torch.ones(t, t, dtype=torch.bool), 1), float("-inf"))
            o = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), vv).reshape(t, -1)
            h = h + o @ a.o_proj.weight.t()
            x = ref.rmsnorm(h, layer.post_attention_layernorm.weight, layer.post_attention_layernorm.eps)
            gu = x @ layer.mlp.gate_up_proj.weight.t()
            gate, up = gu.chunk(2, -1)
            h = h + (torch.nn.functional.silu(gate) * up) @ layer.mlp.down_proj.weight.t()
        h = ref.rmsnorm(h, model.model.norm.weight, model.model.norm.eps)
        return h @ model.lm_head.weight.t()

    want = dense(seq)
    kv = KVCacheManager(cfg, num_pages=8, page_size=16, max_seats=2, max_pages_per_seq=4)
    r = ModelRunner(model, kv)
    pre = r.prefill([0], [seq[:15]])
    assert torch.allclose(pre[0], want[14], atol=2e-4)
    for j in range(15, 21):                                   # token-by-token decode keeps reading the donor's cache
        out = r.step([0], [[seq[j]]])
        assert torch.allclose(out[0], want[j], atol=2e-4)
    # the shared layers' own cache layers were never written
    assert float(kv.pool[2].abs().sum()) == 0.0 and float(kv.pool[3].abs().sum()) == 0.0 and float(kv.pool[1].abs().sum()) > 0


def test_values_from_keys_and_weightless_value_norm():
    """``attention_k_eq_v``: full-attention layers have no value projection and cache the raw key projection as values;
    ``has_value_norm``: values pass a weightless per-head RMSNorm.  Checked against a dense restatement of one layer stack."""
    cfg = tiny_llama_config(num_hidden_layers=2, dtype="float32")
    cfg.attention_k_eq_v, cfg.has_value_norm = True, True
    cfg.layer_windows = [0, 64]                                # layer 0 full attention (k = v), layer 1 sliding (own v_proj)
    model = AutoModel.from_config(cfg, random_init=7)
    a0, a1 = model.model.layers[0].self_attn, model.model.layers[1].self_attn
    assert a0.k_eq_v and not a1.k_eq_v
    assert tuple(a0.qkv_proj.weight.shape) == (cfg.q_size + cfg.kv_size, cfg.hidden_size)
    assert tuple(a1.qkv_proj.weight.shape) == (cfg.q_size + 2 * cfg.kv_size, cfg.hidden_size)
    seq = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(2)).tolist()
    t = len(seq)
    h = model.model.embed_tokens.weight[torch.tensor(seq)]
    cs, pos = model.cos_sin("cpu"), torch.arange(t)
    for layer in model.model.layers:
        a = layer.self_attn
        x = ref.rmsnorm(h, layer.input_layernorm.weight, layer.input_layernorm.eps)
        proj = x @ a.qkv_proj.weight.t()
        if a.k_eq_v:
            q, k = proj.split([cfg.q_size, cfg.kv_size], -1)
            v = k
        else:
            q, k, v = proj.split([cfg.q_size, cfg.kv_size, cfg.kv_size], -1)
        v = v.reshape(t, cfg.num_key_value_heads, cfg.head_dim)
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)
        q = ref.apply_rope(q.reshape(t, cfg.num_attention_heads, cfg.head_dim), pos, cs)
        k = ref.apply_rope(k.reshape(t, cfg.num_key_value_heads, cfg.head_dim), pos, cs)
        rep = cfg.num_attention_heads // cfg.num_key_value_heads
        sc = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(rep, 1)) * cfg.head_dim ** -0.5
        sc = sc.masked_fill(torch.triu(torch.ones(t, t, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), v.repeat_interleave(rep, 1)).reshape(t, -1)
        h = h + o @ a.o_proj.weight.t()
        x = ref.rmsnorm(h, layer.post_attention_layernorm.weight, layer.post_attention_layernorm.eps)
        gate, up = (x @ layer.mlp.gate_up_proj.weight.t()).chunk(2, -1)
        h = h + (torch.nn.functional.silu(gate) * up) @ layer.mlp.down_proj.weight.t()
    want = ref.rmsnorm(h, model.model.norm.weight, model.model.norm.eps) @ model.lm_head.weight.t()
    r = ModelRunner(model, KVCacheManager(cfg, num_pages=4, page_size=16, max_seats=1, max_pages_per_seq=2))
    got = r.prefill([0], [seq[:8]])
    assert torch.allclose(got[0], want[7], atol=2e-4)
    for j in range(8, 12):
        assert torch.allclose(r.step([0], [[seq[j]]])[0], want[j], atol=2e-4)


def test_gemma_checkpoints_with_unbuilt_blocks_are_refused_by_name():
    from tensorrt_edge_llm_b200.config import ModelConfig
    base = {"model_type": "gemma3_text", "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 6, "num_attention_heads": 4,
            "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 300, "sliding_window": 32, "rms_norm_eps": 1e-6, "torch_dtype": "float32"}
    assert ModelConfig.from_hf_dict(base).layer_windows == [32, 32, 32, 32, 32, 0]
    shared = ModelConfig.from_hf_dict({**base, "num_hidden_layers": 12, "sliding_window_pattern": 3, "num_kv_shared_layers": 2,
                                       "attention_k_eq_v": True, "use_value_norm": True})
    assert shared.num_kv_shared_layers == 2 and shared.attention_k_eq_v and shared.has_value_norm
    assert shared.kv_donor(9) == -1 and shared.kv_donor(10) == 9 and shared.kv_donor(11) == 8      # sliding ← sliding, full ← full
    for extra, word in (({"global_head_dim": 32}, "global_head_dim"), ({"hidden_size_per_layer_input": 8}, "per-layer input"),
                        ({"altup_num_inputs": 4}, "AltUp"), ({"num_experts": 8}, "mixture-of-experts")):
        with pytest.raises(NotImplementedError, match=word):
            ModelConfig.from_hf_dict({**base, "model_type": "gemma4_text", **extra})
