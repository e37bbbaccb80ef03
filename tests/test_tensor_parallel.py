"""Tensor parallelism: TP=2 must reproduce TP=1 (CPU ranks over gloo; GPU ranks over NCCL and
over the fused peer-memory communicator when two GPUs are present)."""
import json
import os
import subprocess
import sys

import pytest
import torch

from tensorrt_edge_llm_b200.checkpoint import save_file

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _make_ckpt(d, dtype):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=8, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
                      rope_theta=1e4, max_position_embeddings=1024, tie_word_embeddings=False)
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg).to(dtype).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" not in n:
                p.normal_(0.0, 0.05)
    save_file(dict(m.state_dict()), os.path.join(d, "model.safetensors"))
    hf = cfg.to_dict()
    hf["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)


def _make_moe_ckpt(d, dtype):
    from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM
    cfg = Qwen3MoeConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, moe_intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=8, num_key_value_heads=2, head_dim=128, num_experts=8, num_experts_per_tok=2,
                         norm_topk_prob=True, rms_norm_eps=1e-6, rope_theta=1e4, max_position_embeddings=1024,
                         decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False, output_router_logits=False)
    torch.manual_seed(0)
    m = Qwen3MoeForCausalLM(cfg).to(dtype).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" not in n:
                p.normal_(0.0, 0.05)
    sd = {}
    for k, v in m.state_dict().items():
        if k.endswith("experts.gate_up_proj"):
            base, i = k[:-len(".gate_up_proj")], v.shape[1] // 2
            for e in range(v.shape[0]):
                sd[f"{base}.{e}.gate_proj.weight"], sd[f"{base}.{e}.up_proj.weight"] = v[e, :i].contiguous(), v[e, i:].contiguous()
        elif k.endswith("experts.down_proj"):
            for e in range(v.shape[0]):
                sd[f"{k[:-len('.down_proj')]}.{e}.down_proj.weight"] = v[e].contiguous()
        else:
            sd[k] = v
    save_file(sd, os.path.join(d, "model.safetensors"))
    hf = cfg.to_dict()
    hf["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)


def _launch(nproc, backend, kind, ckpt, port, prompt_len=70, extra=(), env_extra=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "_tp_worker.py"),
           backend, kind, ckpt, str(prompt_len), *extra]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="2", **(env_extra or {}))
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def test_tp2_matches_tp1_cpu_gloo(tmp_path):
    _make_ckpt(str(tmp_path), torch.float32)
    out = _launch(2, "gloo", "nccl", str(tmp_path), 29611)
    assert "ranks identical True" in out


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["nccl", "fused"])
def test_tp2_matches_tp1_gpu(tmp_path, kind):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _make_ckpt(str(tmp_path), torch.bfloat16)
    out = _launch(2, "nccl", kind, str(tmp_path), 29612 if kind == "nccl" else 29613)
    assert "ranks identical True" in out


@pytest.mark.gpu
def test_tp2_fused_prefill_reduce_scatter_path(tmp_path):
    """Prompts long enough (2 x 190 rows) that the row-parallel GEMMs leave through the reduce-scatter
    epilogue and the column-parallel GEMMs wait for the all-gather in their prologue."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _make_ckpt(str(tmp_path), torch.bfloat16)
    out = _launch(2, "nccl", "fused", str(tmp_path), 29614, prompt_len=190)
    assert "ranks identical True" in out


@pytest.mark.gpu
@pytest.mark.parametrize("prompt_len", [30, 70])
def test_tp2_fused_decode_size_reduce_scatter_path(tmp_path, prompt_len):
    """Every step, decode rows included, takes the sharded path: the decode-size GEMM stores its rows into the owner
    rank's buffer from its epilogue and the next one waits for the gathered rows in its producer warp."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _make_ckpt(str(tmp_path), torch.bfloat16)
    out = _launch(2, "nccl", "fused", str(tmp_path), 29618 + (prompt_len > 50), prompt_len=prompt_len, env_extra={"TELB_RS_MIN_ROWS": "1"})
    assert "ranks identical True" in out


@pytest.mark.gpu
@pytest.mark.parametrize("kind,prompt_len,rs_min", [("nccl", 70, "0"), ("fused", 70, "0"), ("fused", 190, "0"), ("fused", 30, "1")])
def test_tp4_matches_tp1_gpu(tmp_path, kind, prompt_len, rs_min):
    """Four ranks: NCCL composition, fused one-shot all-reduce, fused prefill path and the sharded decode-size path."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    _make_ckpt(str(tmp_path), torch.bfloat16)
    port = 29630 + ["nccl70", "fused70", "fused190", "fused30"].index(f"{kind}{prompt_len}")
    out = _launch(4, "nccl", kind, str(tmp_path), port, prompt_len=prompt_len, env_extra={"TELB_RS_MIN_ROWS": rs_min} if rs_min != "0" else None)
    assert "ranks identical True" in out


def test_ep2_matches_single_rank_cpu_gloo(tmp_path):
    """Attention tensor-parallel + experts sharded by id, over gloo: the partial sums reduce to the single-rank model."""
    _make_moe_ckpt(str(tmp_path), torch.float32)
    out = _launch(2, "gloo", "nccl", str(tmp_path), 29615, extra=("ep",))
    assert "ranks identical True" in out


@pytest.mark.gpu
@pytest.mark.parametrize("prompt_len", [70, 190])
def test_ep2_fused_gpu(tmp_path, prompt_len):
    """Expert parallelism on two GPUs: decode-size steps reduce the experts' partial sums in the fused all-reduce;
    prefill-size steps (2 x 190 rows) ship token rows all-to-all over peer memory."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _make_moe_ckpt(str(tmp_path), torch.bfloat16)
    out = _launch(2, "nccl", "fused", str(tmp_path), 29616 + (prompt_len > 100), prompt_len=prompt_len, extra=("ep",))
    assert "ranks identical True" in out


@pytest.mark.gpu
@pytest.mark.parametrize("prompt_len", [30, 190])
def test_ep4_fused_gpu(tmp_path, prompt_len):
    """Expert parallelism on four GPUs (two experts per rank in the test checkpoint): decode-size and prefill-size steps
    through the peer-memory all-to-all, every rank's tokens equal to the single-rank model's."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    _make_moe_ckpt(str(tmp_path), torch.bfloat16)
    out = _launch(4, "nccl", "fused", str(tmp_path), 29640 + (prompt_len > 100), prompt_len=prompt_len, extra=("ep",))
    assert "ranks identical True" in out


@pytest.mark.gpu
def test_fused_allreduce_norm_world1():
    """The fused all-reduce + add + RMSNorm kernel at world size 1 equals the local kernel."""
    from tensorrt_edge_llm_b200.ops import cuda as cu
    import ctypes
    g = torch.Generator(device="cuda").manual_seed(0)
    rows, hidden = 37, 2048
    x = torch.randn(rows, hidden, device="cuda", generator=g).bfloat16()
    r = torch.randn(rows, hidden, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).bfloat16()
    partial = torch.zeros(2 * 256 * hidden, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(2 * 8 * 256, device="cuda", dtype=torch.int32)
    epoch = torch.zeros(256, device="cuda", dtype=torch.int32)
    cp = (ctypes.c_void_p * 1)(partial.data_ptr())
    cf = (ctypes.c_void_p * 1)(flags.data_ptr())
    y, res = torch.empty_like(x), torch.empty_like(x)
    ws = cu.Workspace.get(x.device)
    for _ in range(3):     # epochs advance, buffers alternate
        cu._check(cu.lib().telb_ar_add_rmsnorm(cu._p(x), cp, cf, cu._p(epoch), cu._p(r), cu._p(w), cu._p(res), cu._p(y), None, None,
                                               None, 0, 1, rows, hidden, 256, ctypes.c_float(1e-6), 1, cu._p(ws.status),
                                               cu._stream()), "ar")
    y2, res2 = cu.add_rmsnorm(x, r, w, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(res, res2)
    assert torch.equal(y, y2)
    assert int(epoch[:rows].min()) == 3
    ws.check_status()


def test_in_flight_batching_with_tensor_parallel_ranks_cpu_gloo(tmp_path):
    """Rank 0 schedules (chunked prefill, mid-flight admission), rank 1 replays the mirrored steps; tokens equal TP 1."""
    _make_ckpt(str(tmp_path), torch.float32)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(ROOT, "tests", "_tp_ifb_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0: match True" in r.stdout and "rank 1: followed" in r.stdout
