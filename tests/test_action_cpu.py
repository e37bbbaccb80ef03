"""Flow-matching action expert over the language model's KV cache: one step against a dense restatement, the rollout, and
the trajectory-history tokeniser."""
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.models.action_expert import ActionConfig, ActionExpert
from tensorrt_edge_llm_b200.ops import reference as ref
from tensorrt_edge_llm_b200.runtime.action import ActionRunner, trajectory_to_token_ids
from tensorrt_edge_llm_b200.runtime.block_diffusion import full_mask
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


def _setup(tokens=6):
    tcfg = tiny_llama_config(num_hidden_layers=3, vocab_size=120, dtype="float32", num_key_value_heads=2, head_dim=16)
    target = AutoModel.from_config(tcfg, random_init=0)
    kv = KVCacheManager(tcfg, num_pages=24, page_size=16, max_seats=2, max_pages_per_seq=6)
    runner = ModelRunner(target, kv)
    ac = ActionConfig(hidden_size=32, intermediate_size=48, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                      rope_theta=10000.0, n_diffusion_tokens=tokens, in_proj_hidden_size=24, in_proj_num_fourier_feats=8, in_proj_max_freq=2.0, dtype="float32")
    expert = ActionExpert(ac).init_random(3, std=0.1)       # low frequencies, small weights: rounding differences stay small over steps
    return runner, expert, tcfg


def test_one_step_matches_dense_attention_over_the_model_cache():
    runner, expert, tcfg = _setup()
    prompt = [5, 6, 7, 8, 9, 10, 11, 12, 13]
    runner.prefill([0], [prompt])
    n, t = len(prompt), 6
    x = torch.randn(1, t, 2, generator=torch.Generator().manual_seed(1))
    meta = runner._meta([0], [t], tree_mask=full_mask(t, t, "cpu"))
    got = expert.velocity(x, torch.tensor([0.3]), meta, runner.cache)
    # dense restatement, layer by layer
    h = expert.action_in_proj(x, torch.tensor([0.3]))
    cs = expert.cos_sin("cpu")
    pos = torch.arange(n, n + t)
    for i, layer in enumerate(expert.layers):
        a = layer.self_attn
        xin = ref.rmsnorm(h, layer.input_layernorm.weight, layer.input_layernorm.eps)
        qkv = xin @ a.qkv_proj.weight.T
        q, k, v = qkv.split([a.num_q_heads * 16, a.num_kv_heads * 16, a.num_kv_heads * 16], -1)
        q = ref.apply_rope(ref._head_rmsnorm(q.reshape(t, -1, 16), a.q_norm.weight, a.eps), pos, cs)
        k = ref.apply_rope(ref._head_rmsnorm(k.reshape(t, -1, 16), a.k_norm.weight, a.eps), pos, cs)
        kc, vc = ref.gather_kv(runner.cache[i], runner.kv.table_rows([0])[0], n, 16)          # the language model's own keys
        kk = torch.cat([kc, k.permute(1, 0, 2)], 1)                                            # [Hkv, n + t, D]
        vv = torch.cat([vc, v.reshape(t, -1, 16).permute(1, 0, 2)], 1)
        rep = a.num_q_heads // a.num_kv_heads
        att = torch.softmax(torch.einsum("thd,hsd->hts", q, kk.repeat_interleave(rep, 0)) * 16 ** -0.5, -1)
        o = torch.einsum("hts,hsd->thd", att, vv.repeat_interleave(rep, 0)).reshape(t, -1)
        h = h + o @ a.o_proj.weight.T
        xin = ref.rmsnorm(h, layer.post_attention_layernorm.weight, layer.post_attention_layernorm.eps)
        gu = xin @ layer.mlp.gate_up_proj.weight.T
        inter = gu.shape[-1] // 2
        h = h + (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]) @ layer.mlp.down_proj.weight.T
    want = expert.action_out_proj(ref.rmsnorm(h, expert.norm.weight, expert.norm.eps)).reshape(1, t, 2)
    assert (got - want).abs().max() < 1e-4
    assert runner.kv.lengths[0] == n                                   # nothing committed


def test_rollout_is_euler_integration_and_leaves_the_cache_usable():
    runner, expert, tcfg = _setup()
    prompts = [[5, 6, 7, 8, 9], [20, 21, 22, 23, 24, 25, 26]]
    logits = runner.prefill([0, 1], prompts)
    before = runner.step([0, 1], [[int(logits[0].argmax())], [int(logits[1].argmax())]], commit=False).clone()
    act = ActionRunner(runner, expert, num_steps=4)
    noise = torch.randn(2, 6, 2, generator=torch.Generator().manual_seed(2))
    traj = act.sample([0, 1], noise=noise)
    assert traj.shape == (2, 6, 2) and runner.kv.lengths[0] == 5 and runner.kv.lengths[1] == 7
    # by hand: four Euler steps with the same velocity calls
    x = noise.clone()
    for i in range(4):
        meta = runner._meta([0, 1], [6, 6], tree_mask=full_mask(12, 6, "cpu"))
        x = x + 0.25 * expert.velocity(x, torch.full((2,), i / 4), meta, runner.cache)
    assert (traj - x).abs().max() < 1e-5
    # sequences do not influence each other, and the seed decides the noise
    solo = act.sample([1], noise=noise[1:])
    assert (solo[0] - traj[1]).abs().max() < 1e-4
    assert torch.equal(act.sample([0], seed=7), act.sample([0], seed=7)) and not torch.equal(act.sample([0], seed=7), act.sample([0], seed=8))
    # the language model carries on as if nothing happened
    after = runner.step([0, 1], [[int(logits[0].argmax())], [int(logits[1].argmax())]], commit=False)
    assert torch.equal(before, after)


def test_geometry_must_match_and_history_tokens():
    runner, expert, tcfg = _setup()
    bad = ActionExpert(ActionConfig(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                    head_dim=16, n_diffusion_tokens=4, in_proj_hidden_size=24, in_proj_num_fourier_feats=8, dtype="float32"))
    try:
        ActionRunner(runner, bad)
        raise AssertionError("layer mismatch accepted")
    except ValueError:
        pass
    ids = trajectory_to_token_ids([(0.0, 0.0, 0.0), (1.0, -0.5, 0.0), (9.0, -0.5, 0.0)], 1000, 3000)
    # first point absolute (centre of every range), then steps: (+1, -0.5, 0) and (+8 → clamped to +4, 0, 0)
    assert ids[:3] == [3000 + 500, 3000 + 500, 3000 + 500]
    assert ids[3:6] == [3000 + round(5 / 8 * 999), 3000 + round(3.5 / 8 * 999), 3000 + 500]
    assert ids[6:] == [3000 + 999, 3000 + 500, 3000 + 500]
    # checkpoint names of the reference layout map onto the modules
    assert ActionExpert.checkpoint_key_remap("expert.layers.2.mlp_gate_proj.weight") == "layers.2.mlp.gate_proj.weight"
    assert ActionExpert.checkpoint_key_remap("expert.layers.0.self_attn.q_norm.weight") == "layers.0.self_attn.q_norm.weight"
    assert ActionExpert.checkpoint_key_remap("action_out_proj.bias") == "action_out_proj.bias"


def test_expert_checkpoint_roundtrip_and_command(tmp_path):
    """Save an expert under the reference's tensor names, load it back, and run the command's library form."""
    import json
    import os
    from tensorrt_edge_llm_b200.checkpoint import save_file
    from tensorrt_edge_llm_b200.commands.action import run_requests
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    runner, expert, tcfg = _setup()
    sd = {}
    for name, t in expert.state_dict().items():
        if name.startswith("layers."):
            name = "expert." + name.replace(".mlp.down_proj.", ".mlp_down_proj.")
        elif name == "norm.weight":
            name = "expert.norm.weight"
        name = name.replace("action_in_proj.encoder.", "action_in_proj.encoder.trunk.")
        sd[name] = t.contiguous()
    # the fused projections go back to the per-projection tensors a checkpoint holds
    for i, layer in enumerate(expert.layers):
        a = layer.self_attn
        q, k, v = a.qkv_proj.weight.split([a.num_q_heads * 16, a.num_kv_heads * 16, a.num_kv_heads * 16], 0)
        g, u = layer.mlp.gate_up_proj.weight.chunk(2, 0)
        for n, t in (("self_attn.q_proj", q), ("self_attn.k_proj", k), ("self_attn.v_proj", v), ("mlp_gate_proj", g), ("mlp_up_proj", u)):
            sd[f"expert.layers.{i}.{n}.weight"] = t.contiguous()
        sd.pop(f"expert.layers.{i}.self_attn.qkv_proj.weight")
        sd.pop(f"expert.layers.{i}.mlp.gate_up_proj.weight")
    d = str(tmp_path)
    save_file(sd, os.path.join(d, "model.safetensors"))
    json.dump({"action_config": dict(vars(expert.action_cfg))}, open(os.path.join(d, "config.json"), "w"))
    loaded = ActionExpert.from_pretrained(d)
    x = torch.randn(1, 6, 2, generator=torch.Generator().manual_seed(3))
    runner.prefill([0], [[5, 6, 7, 8]])
    meta = runner._meta([0], [6], tree_mask=full_mask(6, 6, "cpu"))
    assert torch.allclose(loaded.velocity(x, torch.tensor([0.5]), meta, runner.cache), expert.velocity(x, torch.tensor([0.5]), meta, runner.cache),
                          atol=1e-6)
    llm = LLM(tcfg, device="cpu", max_batch_size=1, max_input_len=64, max_kv_cache_capacity=128, page_size=16)
    body = {"requests": [{"prompt_token_ids": [5, 6, 7, 8, 9], "trajectory_history": [[0, 0, 0], [0.5, 0.1, 0]], "max_generate_length": 5, "seed": 3},
                         {"prompt_token_ids": [9, 8, 7], "max_generate_length": 3}]}
    expert.action_cfg.num_traj_tokens, expert.action_cfg.traj_token_start = 20, 90
    res = run_requests(llm, expert, body, num_steps=3)
    assert len(res) == 2 and len(res[0]["token_ids"]) == 5 and len(res[0]["trajectory"]) == 6 and len(res[0]["trajectory"][0]) == 2
    again = run_requests(llm, expert, body, num_steps=3)
    assert again == res                                              # seeded noise: the same trajectories
    from tensorrt_edge_llm_b200 import cli
    assert "action" in cli.COMMANDS
