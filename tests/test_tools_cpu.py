"""Command-line tools on CPU: quantise-and-reload, LoRA processing / merging, vocabulary reduction, build check."""
import json
import os

import pytest
import torch

from tensorrt_edge_llm_b200 import AutoModel
from tensorrt_edge_llm_b200.checkpoint import save_file
from tensorrt_edge_llm_b200.checkpoint.safetensors_io import SafetensorsFile
from tensorrt_edge_llm_b200.cli import main as trtedge
from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
from tensorrt_edge_llm_b200.runtime.runner import ModelRunner


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    from transformers import LlamaConfig, LlamaForCausalLM
    d = str(tmp_path_factory.mktemp("ckpt"))
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, rope_theta=1e4, max_position_embeddings=256,
                      tie_word_embeddings=False, bos_token_id=1, eos_token_id=2)
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg).float().eval()
    save_file(dict(m.state_dict()), os.path.join(d, "model.safetensors"))
    hf = cfg.to_dict()
    hf["torch_dtype"] = "float32"
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    return d


def _logits(model_dir, ids):
    model = AutoModel.from_pretrained(model_dir)
    kv = KVCacheManager(model.cfg, num_pages=8, page_size=16, max_seats=2, max_pages_per_seq=4)
    return ModelRunner(model, kv).prefill([0], [ids]).float()


def test_quantize_nvfp4_and_reload(ckpt, tmp_path):
    out = str(tmp_path / "q")
    assert trtedge(["quantize", "llm", "--model_dir", ckpt, "--output_dir", out, "--quantization", "nvfp4"]) == 0
    qc = json.load(open(os.path.join(out, "hf_quant_config.json")))["quantization"]
    assert qc["quant_algo"] == "NVFP4" and qc["group_size"] == 16 and "lm_head" in qc["exclude_modules"]
    f = SafetensorsFile(os.path.join(out, "model.safetensors"))
    base = "model.layers.0.self_attn.q_proj"
    assert f.info(base + ".weight") == (torch.uint8, [128, 64]) and f.info(base + ".weight_scale")[0] == torch.float8_e4m3fn
    assert f.info(base + ".input_scale")[1] == [] and f.info("lm_head.weight")[0] == torch.float32
    # q/k/v read the same activations, so calibration gives them one input scale
    assert float(f.get(base + ".input_scale")) == float(f.get("model.layers.0.self_attn.k_proj.input_scale")) > 0
    ids = list(range(5, 45))
    a, b = _logits(ckpt, ids), _logits(out, ids)
    cos = torch.nn.functional.cosine_similarity(a - a.mean(), b - b.mean(), dim=-1)
    assert float(cos) > 0.95                      # 4-bit weights and activations on a tiny random model


def test_quantize_int4_awq(ckpt, tmp_path):
    out = str(tmp_path / "q4")
    assert trtedge(["quantize", "--model_dir", ckpt, "--output_dir", out, "--quantization", "int4_awq", "--group-size", "64"]) == 0
    f = SafetensorsFile(os.path.join(out, "model.safetensors"))
    assert f.info("model.layers.1.mlp.down_proj.weight") == (torch.uint8, [64, 256])
    assert f.info("model.layers.1.mlp.down_proj.weight_scale")[1] == [128, 4]
    ids = list(range(5, 45))
    a, b = _logits(ckpt, ids), _logits(out, ids)
    assert float(torch.nn.functional.cosine_similarity(a - a.mean(), b - b.mean(), dim=-1)) > 0.97


def _adapter(d, r=4, alpha=8.0):
    os.makedirs(d, exist_ok=True)
    g = torch.Generator().manual_seed(1)
    t = {}
    for mod, (o, i) in {"model.layers.0.self_attn.q_proj": (128, 128), "model.layers.1.mlp.down_proj": (128, 256)}.items():
        t[f"base_model.model.{mod}.lora_A.weight"] = torch.randn(r, i, generator=g) * 0.1
        t[f"base_model.model.{mod}.lora_B.weight"] = torch.randn(o, r, generator=g) * 0.1
    save_file(t, os.path.join(d, "adapter_model.safetensors"))
    with open(os.path.join(d, "adapter_config.json"), "w") as f:
        json.dump({"r": r, "lora_alpha": alpha, "target_modules": ["q_proj", "down_proj"]}, f)
    return t


def test_lora_process_and_merge(ckpt, tmp_path):
    ad = str(tmp_path / "adapter")
    t = _adapter(ad)
    out = str(tmp_path / "lora_rt")
    assert trtedge(["process-lora", "--input_dir", ad, "--output_dir", out]) == 0
    f = SafetensorsFile(os.path.join(out, "lora_weights.safetensors"))
    b = f.get("lora_B_model.layers.0.self_attn.q_proj").float()
    assert torch.allclose(b, (t["base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight"] * 2.0).half().float())
    assert json.load(open(os.path.join(out, "lora_config.json")))["rank"] == 4
    merged = str(tmp_path / "merged")
    assert trtedge(["merge-lora", "--model_dir", ckpt, "--lora_dir", ad, "--output_dir", merged]) == 0
    w0 = SafetensorsFile(os.path.join(ckpt, "model.safetensors")).get("model.layers.1.mlp.down_proj.weight")
    w1 = SafetensorsFile(os.path.join(merged, "model.safetensors")).get("model.layers.1.mlp.down_proj.weight")
    delta = 2.0 * t["base_model.model.model.layers.1.mlp.down_proj.lora_B.weight"] @ t["base_model.model.model.layers.1.mlp.down_proj.lora_A.weight"]
    assert torch.allclose(w1 - w0, delta, atol=1e-5)
    assert trtedge(["insert-lora", "--lora_dir", ad]) == 0
    assert not torch.allclose(_logits(ckpt, [3, 4, 5]), _logits(merged, [3, 4, 5]))


def test_insert_lora_declares_slots_the_runtime_reserves(ckpt, tmp_path, capsys):
    import shutil
    from tensorrt_edge_llm_b200.lora.runtime import LoraLinear
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    ad, rt_dir = str(tmp_path / "adapter"), str(tmp_path / "rt")
    _adapter(ad)
    model_dir = str(tmp_path / "model")
    shutil.copytree(ckpt, model_dir)
    assert trtedge(["insert-lora", "--lora_dir", ad, "--model_dir", model_dir, "--max-lora-rank", "8"]) == 0
    decl = json.load(open(os.path.join(model_dir, "lora_slots.json")))
    assert decl["max_lora_rank"] == 8 and decl["slots"]["model.layers.0.self_attn.q_proj"]["module"].endswith("self_attn.qkv_proj")
    assert decl["slots"]["model.layers.0.self_attn.q_proj"]["source"] == 0 and decl["slots"]["model.layers.1.mlp.down_proj"]["in_features"] == 256
    # an adapter that does not fit the model is refused and leaves the declaration alone
    bad = str(tmp_path / "bad")
    _adapter(bad)
    f = SafetensorsFile(os.path.join(bad, "adapter_model.safetensors"))
    t = {k: f.get(k).clone() for k in f.keys()}
    t["base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight"] = torch.zeros(4, 64)
    save_file(t, os.path.join(bad, "adapter_model.safetensors"))
    assert trtedge(["insert-lora", "--lora_dir", bad, "--model_dir", model_dir]) == 1
    assert "do not fit" in capsys.readouterr().out
    # the runtime wraps the declared layers at load and enforces the declared rank
    llm = LLM(model_dir, device="cpu", max_batch_size=1, max_input_len=64, max_kv_cache_capacity=96)
    assert llm.lora is not None and isinstance(llm.model.model.layers[0].self_attn.qkv_proj, LoraLinear)
    assert isinstance(llm.model.model.layers[1].mlp.down_proj, LoraLinear) and not isinstance(llm.model.model.layers[0].mlp.down_proj, LoraLinear)
    assert trtedge(["process-lora", "--input_dir", ad, "--output_dir", rt_dir]) == 0
    llm.load_lora("style", rt_dir)
    llm.lora.max_rank = 2
    with pytest.raises(ValueError, match="rank"):
        llm.load_lora("other", rt_dir)
    llm.close()


def test_lora_runtime_adapter_equals_merged_checkpoint(ckpt, tmp_path):
    from tensorrt_edge_llm_b200.lora import LoraManager
    ad, rt_dir, merged = str(tmp_path / "adapter"), str(tmp_path / "rt"), str(tmp_path / "merged")
    _adapter(ad)
    assert trtedge(["process-lora", "--input_dir", ad, "--output_dir", rt_dir, "--dtype", "bfloat16"]) == 0
    assert trtedge(["merge-lora", "--model_dir", ckpt, "--lora_dir", ad, "--output_dir", merged]) == 0
    ids = list(range(5, 40))
    model = AutoModel.from_pretrained(ckpt)
    mgr = LoraManager(model)
    mgr.load_adapter("style", rt_dir)
    kv = KVCacheManager(model.cfg, num_pages=8, page_size=16, max_seats=2, max_pages_per_seq=4)
    r = ModelRunner(model, kv)
    base = r.prefill([0], [ids]).float()
    kv.free(0)
    mgr.set_active("style")
    adapted = r.prefill([0], [ids]).float()
    kv.free(0)
    mgr.set_active(None)
    again = r.prefill([0], [ids]).float()
    want = _logits(merged, ids)
    assert torch.allclose(base, again) and not torch.allclose(base, adapted, atol=1e-4)
    assert (adapted - want).abs().max() < 2e-2 * want.abs().max()          # adapter weights are stored in bf16
    with pytest.raises(KeyError):
        mgr.set_active("missing")


def test_reduce_vocab(ckpt, tmp_path):
    corpus = str(tmp_path / "ids.json")
    json.dump([[7, 7, 7, 9, 9, 400], [9, 400, 400, 400, 11]], open(corpus, "w"))
    out = str(tmp_path / "rv")
    assert trtedge(["reduce-vocab", "--model_dir", ckpt, "--output_dir", out, "--keep", "5", "--corpus-ids", corpus]) == 0
    f = SafetensorsFile(os.path.join(out, "vocab_map.safetensors"))
    vm = f.get("vocab_map").tolist()
    assert vm == [1, 2, 7, 9, 400]                 # bos / eos forced, then the three most frequent
    head = SafetensorsFile(os.path.join(ckpt, "model.safetensors")).get("lm_head.weight")
    assert torch.equal(f.get("lm_head.weight"), head[vm])
    from tensorrt_edge_llm_b200.vocab_reduction import map_to_full
    assert map_to_full(torch.tensor([4, 0]), torch.tensor(vm)).tolist() == [400, 1]


def test_reduced_vocab_at_run_time(ckpt, tmp_path):
    """An LLM opened on a directory that holds ``vocab_map.safetensors`` runs the reduced head and returns full-vocabulary ids."""
    import shutil
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    from tensorrt_edge_llm_b200.vocab_reduction import reduce_vocab
    prompts = [[5, 9, 33, 70], [8, 2, 44]]
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    full = [o.token_ids for o in LLM(ckpt, max_batch_size=2, max_kv_cache_capacity=128, device="cpu").generate(prompts, sp)]
    vocab = AutoModel.from_pretrained(ckpt).cfg.vocab_size
    # every token kept, in a shuffled order: the outputs must not change
    perm_dir = str(tmp_path / "perm")
    shutil.copytree(ckpt, perm_dir)
    reduce_vocab(ckpt, perm_dir, torch.randperm(vocab, generator=torch.Generator().manual_seed(1)))
    llm = LLM(perm_dir, max_batch_size=2, max_kv_cache_capacity=128, device="cpu")
    assert llm.model.lm_head.out_features == vocab
    assert [o.token_ids for o in llm.generate(prompts, sp)] == full
    # a strict subset: every generated id lies in it, with and without in-flight batching
    sub_dir = str(tmp_path / "sub")
    shutil.copytree(ckpt, sub_dir)
    keep = torch.arange(3, vocab, 7)
    reduce_vocab(ckpt, sub_dir, keep)
    allowed = set(keep.tolist())
    for ifb in (False, True):
        llm = LLM(sub_dir, max_batch_size=2, max_kv_cache_capacity=128, device="cpu", enable_in_flight_batching=ifb)
        assert llm.model.lm_head.out_features == keep.numel()
        for o in llm.generate(prompts, SamplingParams(max_tokens=6, temperature=0.8, top_k=20, seed=3)):
            assert len(o.token_ids) > 0 and set(o.token_ids) <= allowed


def test_build_checks_checkpoint(ckpt, tmp_path):
    out = str(tmp_path / "built")
    assert trtedge(["build", ckpt, "--output_dir", out, "--tensor-parallel-size", "2", "--max-batch-size", "4"]) == 0
    rc = json.load(open(os.path.join(out, "runtime_config.json")))
    assert rc["deployment"]["tensor_parallel_size"] == 2 and rc["model"]["hidden_size"] == 128
    broken = str(tmp_path / "broken")
    os.makedirs(broken)
    f = SafetensorsFile(os.path.join(ckpt, "model.safetensors"))
    save_file({k: f.get(k).clone() for k in f.keys() if "layers.1.mlp.up_proj" not in k}, os.path.join(broken, "model.safetensors"))
    json.dump(json.load(open(os.path.join(ckpt, "config.json"))), open(os.path.join(broken, "config.json"), "w"))
    assert trtedge(["build", broken]) == 1
    assert trtedge(["--version"]) == 0 and trtedge([]) == 2


def test_build_writes_artifacts_that_load_without_repacking(ckpt, tmp_path):
    """`trtedge build` prepares per-rank weights + world / runtime configs; the directory then stands in for the checkpoint:
    same tensors as a direct sharded load on every rank, same tokens through `LLM`, tampering is detected on request."""
    from tensorrt_edge_llm_b200 import AutoModel
    from tensorrt_edge_llm_b200.checkpoint.artifacts import is_artifact_dir, load_artifacts, read_world_config
    from tensorrt_edge_llm_b200.config import Mapping
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams
    out2 = str(tmp_path / "tp2")
    assert trtedge(["build", ckpt, "--output_dir", out2, "--tensor-parallel-size", "2"]) == 0
    world = read_world_config(out2)
    assert is_artifact_dir(out2) and world["tensor_parallel_size"] == 2 and [r["weights"] for r in world["ranks"]] == ["rank0.safetensors", "rank1.safetensors"]
    for rank in range(2):
        direct = AutoModel.from_pretrained(ckpt, mapping=Mapping(tp_size=2, tp_rank=rank))
        loaded = AutoModel.from_pretrained(out2, mapping=Mapping(tp_size=2, tp_rank=rank))
        a, b = direct.state_dict(), loaded.state_dict()
        assert a.keys() == b.keys()
        assert [k for k in a if not torch.equal(a[k], b[k])] == []
    with pytest.raises(ValueError, match="tensor-parallel"):
        AutoModel.from_pretrained(out2)                                   # prepared for two ranks, asked for one
    out1 = str(tmp_path / "tp1")
    assert trtedge(["build", ckpt, "--output_dir", out1, "--max-batch-size", "2"]) == 0
    prompts, sp = [[5, 9, 33, 70], [8, 2, 44]], SamplingParams(max_tokens=6)
    want = [o.token_ids for o in LLM(ckpt, max_batch_size=2, max_kv_cache_capacity=128, device="cpu").generate(prompts, sp)]
    got = [o.token_ids for o in LLM(out1, max_batch_size=2, max_kv_cache_capacity=128, device="cpu").generate(prompts, sp)]
    assert got == want
    # a flipped byte in the weight file is caught when verification is requested
    path = os.path.join(out1, "rank0.safetensors")
    raw = bytearray(open(path, "rb").read())
    raw[-1] ^= 0xFF
    open(path, "wb").write(bytes(raw))
    with pytest.raises(ValueError, match="sha256"):
        load_artifacts(out1, verify=True)


def test_reference_package_name_resolves():
    import tensorrt_edgellm
    from tensorrt_edgellm.server import LLM, SamplingParams  # noqa: F401
    from tensorrt_edgellm.config import ModelConfig, QuantConfig  # noqa: F401
    assert tensorrt_edgellm.AutoModel is AutoModel and "serve" in tensorrt_edgellm.cli.COMMANDS


@pytest.mark.parametrize("fmt", ["gptq", "awq", "fp8", "int8_sq", "mxfp8", "q8_0"])
def test_weight_only_checkpoint_formats_load(ckpt, tmp_path, fmt):
    """A checkpoint whose linears are stored as GPTQ / AutoAWQ / FP8 / INT8-SQ / MXFP8 / Q8_0 loads and tracks the 16-bit model."""
    from tensorrt_edge_llm_b200.checkpoint import repacking as R
    enc = {"gptq": lambda w: R.encode_gptq(w, 64), "awq": lambda w: R.encode_autoawq(w, 64), "fp8": R.encode_fp8,
           "int8_sq": R.encode_int8_sq, "mxfp8": R.encode_mxfp8, "q8_0": R.encode_q8_0}[fmt]
    qcfg = {"gptq": {"quant_method": "gptq", "bits": 4, "group_size": 64}, "awq": {"quant_method": "awq", "bits": 4, "group_size": 64},
            "fp8": {"quant_method": "fp8"}, "int8_sq": {"quant_algo": "W8A8_SQ_PER_CHANNEL"}, "mxfp8": {"quant_algo": "MXFP8"},
            "q8_0": {"quant_algo": "Q8_0"}}[fmt]
    out = str(tmp_path / fmt)
    os.makedirs(out)
    f = SafetensorsFile(os.path.join(ckpt, "model.safetensors"))
    tensors = {}
    for k in f.keys():
        t = f.get(k).clone()
        if k.endswith("_proj.weight"):
            base = k[:-len("weight")]
            for name, v in enc(t).items():
                tensors[base + name] = v.reshape(-1) if v.dim() == 0 else v
        else:
            tensors[k] = t
    save_file(tensors, os.path.join(out, "model.safetensors"))
    hf = json.load(open(os.path.join(ckpt, "config.json")))
    hf["quantization_config"] = {**qcfg, "modules_to_not_convert": ["lm_head"]}
    json.dump(hf, open(os.path.join(out, "config.json"), "w"))
    ids = [5, 9, 33, 70, 12, 8]
    a, b = _logits(ckpt, ids), _logits(out, ids)
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0)
    assert float(cos) > (0.97 if fmt in ("gptq", "awq") else 0.995)
    from tensorrt_edge_llm_b200.models.linear import ExpandedLinear
    m = AutoModel.from_pretrained(out)
    assert sum(isinstance(x, ExpandedLinear) for x in m.modules()) >= 7 * m.cfg.num_hidden_layers - 7


def test_quantize_command_other_formats(ckpt, tmp_path):
    ids = [5, 9, 33, 70, 12, 8]
    a = _logits(ckpt, ids)
    for q in ("fp8", "q8_0", "int4_gptq"):
        out = str(tmp_path / q)
        assert trtedge(["quantize", "llm", "--model_dir", ckpt, "--output_dir", out, "--quantization", q, "--group-size", "64"]) == 0
        cos = torch.nn.functional.cosine_similarity(a.flatten(), _logits(out, ids).flatten(), dim=0)
        assert float(cos) > 0.97


def test_request_file_parsing_and_run():
    from tensorrt_edge_llm_b200.chat_template import ChatTemplate
    from tensorrt_edge_llm_b200.commands.infer import RequestFileError, parse_request_file, run_requests
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    body = {"temperature": 0.0, "max_generate_length": 5, "num_logprobs": 2, "logit_bias": {"7": -100},
            "requests": [{"messages": [{"role": "user", "content": "hi"}]},
                         {"messages": [{"role": "user", "content": [{"type": "text", "text": "yo"}]}], "num_logprobs": 0, "logit_bias": {"9": 100},
                          "guided_decoding": {"choice": ["ab", "cd"]}, "stop": "b", "sampling_seed": 7}]}
    reqs = parse_request_file(body)
    assert reqs[0]["num_logprobs"] == 2 and reqs[0]["logit_bias"] == {7: -100.0} and reqs[0]["guided"] is None and reqs[0]["seed"] == 42
    assert reqs[1]["num_logprobs"] == 0 and reqs[1]["logit_bias"] == {9: 100.0} and reqs[1]["guided"].type == "choice" and reqs[1]["seed"] == 7
    for bad in ({}, {"requests": []}, {"requests": [{"messages": [{"role": "robot", "content": "x"}]}]},
                {"requests": [{"messages": [{"role": "user", "content": "x"}], "num_logprobs": 51}]},
                {"requests": [{"messages": [{"role": "user", "content": "x"}], "guided_decoding": {"regex": "a", "choice": ["b"]}}]}):
        with pytest.raises(RequestFileError):
            parse_request_file(bad)

    class Bytes:
        def encode(self, text, add_special_tokens=False):
            return [b + 3 for b in text.encode("utf-8")]

        def decode(self, ids, skip_special_tokens=True):
            return bytes((i - 3) % 256 for i in ids).decode("utf-8", "replace")

        def id_to_bytes(self, i):
            return bytes([(i - 3) % 256])
    llm = LLM(tiny_llama_config(num_hidden_layers=1, vocab_size=300), device="cpu", max_batch_size=1, max_input_len=128, max_kv_cache_capacity=192,
              page_size=16, tokenizer=Bytes())
    reqs[1]["logit_bias"] = None
    res = run_requests(llm, ChatTemplate(), reqs)
    assert res[0]["output_tokens"] == 5 and len(res[0]["logprobs"]) == 5 and len(res[0]["logprobs"][0]["top"]) == 2
    assert res[1]["output_text"] in ("a", "cd") and "logprobs" not in res[1]             # "ab" is cut at the stop string
    llm.close()


def test_lora_per_request_under_in_flight_batching(ckpt, tmp_path):
    """Requests of one batch choose different adapters (or none); each gets the tokens of a run with only its adapter."""
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    a1, a2, r1, r2 = (str(tmp_path / n) for n in ("a1", "a2", "r1", "r2"))
    _adapter(a1, r=4, alpha=64.0)
    torch.manual_seed(77)
    _adapter(a2, r=2, alpha=64.0)
    assert trtedge(["process-lora", "--input_dir", a1, "--output_dir", r1, "--dtype", "bfloat16"]) == 0
    assert trtedge(["process-lora", "--input_dir", a2, "--output_dir", r2, "--dtype", "bfloat16"]) == 0
    prompts = [[5, 9, 33, 70, 12], [8, 2, 44, 19], [7, 7, 3, 50, 61, 4]]
    kw = dict(max_batch_size=3, max_kv_cache_capacity=128, page_size=16, device="cpu")

    def solo(name):
        llm = LLM(ckpt, **kw)
        llm.load_lora("one", r1)
        llm.load_lora("two", r2)
        outs = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=6, lora_name=name, ignore_eos=True))]
        llm.close()
        return outs
    base, one, two = solo(None), solo("one"), solo("two")
    assert base != one and base != two and one != two
    ifb = LLM(ckpt, enable_in_flight_batching=True, **kw)
    ifb.load_lora("one", r1)
    ifb.load_lora("two", r2)
    hs = [ifb.submit(p, SamplingParams(max_tokens=6, lora_name=n, ignore_eos=True)) for p, n in zip(prompts, ("one", None, "two"))]
    from tensorrt_edge_llm_b200.lora.runtime import LoraLinear
    calls0 = LoraLinear.grouped_calls
    got = [h.get(60.0) for h in hs]
    assert got == [one[0], base[1], two[2]]
    assert LoraLinear.grouped_calls > calls0            # steps that mixed both adapters ran the stacked two-GEMM form
    with pytest.raises(ValueError):
        ifb.submit(prompts[0], SamplingParams(max_tokens=2, lora_name="three"))
    # the per-segment form gives the same tokens
    for w in ifb.lora._wrapped.values():
        w.grouped = False
    hs = [ifb.submit(p, SamplingParams(max_tokens=6, lora_name=n, ignore_eos=True)) for p, n in zip(prompts, ("one", None, "two"))]
    assert [h.get(60.0) for h in hs] == got
    ifb.close()


def test_prefix_cache_is_keyed_by_adapter(ckpt, tmp_path):
    """The same prompt under adapter "one" and then under the base model: the second request must not adopt the first one's
    KV pages (LoRA wraps the QKV projection, so their K/V differ) and must produce the tokens of a run without the cache."""
    from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams
    a1, r1 = str(tmp_path / "a1"), str(tmp_path / "r1")
    _adapter(a1, r=4, alpha=64.0)
    assert trtedge(["process-lora", "--input_dir", a1, "--output_dir", r1, "--dtype", "bfloat16"]) == 0
    prompt = [(7 * i + 3) % 90 + 5 for i in range(41)]               # two full 16-token pages + a tail
    kw = dict(max_batch_size=2, max_kv_cache_capacity=128, page_size=16, device="cpu", enable_in_flight_batching=True)

    def run(llm, name):
        return llm.submit(prompt, SamplingParams(max_tokens=6, lora_name=name, ignore_eos=True)).get(60.0)
    plain = LLM(ckpt, **kw)
    plain.load_lora("one", r1)
    want_one, want_base = run(plain, "one"), run(plain, None)
    plain.close()
    assert want_one != want_base
    llm = LLM(ckpt, enable_prefix_cache=True, **kw)
    llm.load_lora("one", r1)
    pc = llm.session.prefix
    assert run(llm, "one") == want_one
    hits0 = pc.hits
    assert run(llm, None) == want_base and pc.hits == hits0          # base model: no hit on the adapter's pages
    assert run(llm, None) == want_base and pc.hits == hits0 + 1      # ... but on its own
    assert run(llm, "one") == want_one and pc.hits == hits0 + 2
    llm.load_lora("one", r1)                                         # reloaded under the same name: a new identity
    assert run(llm, "one") == want_one and pc.hits == hits0 + 2
    llm.close()


def test_runtime_names_of_the_reference_package():
    """``tensorrt_edgellm.runtime`` carries the reference's runtime class names; ``LLMRuntime`` answers a request file,
    counts prompt tokens and opens a stepped session over the same model."""
    import tensorrt_edgellm.runtime as rt_names
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    for name in ("LLMRuntime", "RequestEngine", "RequestHandle", "StreamChannel", "MultiStageRuntime", "validate_scheduling_options"):
        assert getattr(rt_names, name) is not None

    class Bytes:
        def encode(self, text, add_special_tokens=False):
            return [b + 3 for b in text.encode("utf-8")]

        def decode(self, ids, skip_special_tokens=True):
            return bytes((i - 3) % 256 for i in ids).decode("utf-8", "replace")

        def id_to_bytes(self, i):
            return bytes([(i - 3) % 256])
    llm = LLM(tiny_llama_config(num_hidden_layers=1, vocab_size=300), device="cpu", max_batch_size=2, max_input_len=128,
              max_kv_cache_capacity=192, page_size=16, tokenizer=Bytes())
    runtime = rt_names.LLMRuntime(None, llm=llm)
    body = {"temperature": 0.0, "max_generate_length": 4, "requests": [{"messages": [{"role": "user", "content": "hi"}]},
                                                                           {"messages": [{"role": "user", "content": "hello there"}]}]}
    out = runtime.handle_request(body)
    assert [r["output_tokens"] for r in out["responses"]] == [4, 4]
    counts = runtime.count_prompt_tokens(json.dumps(body))
    assert counts[1] > counts[0] > 0 and counts == [r["input_tokens"] for r in out["responses"]]
    assert runtime.max_batch_size() == 2 and runtime.world_size() == 1 and runtime.owns_global_rank(0) and not runtime.has_draft_model()
    assert runtime.unavailable_reason() == "" and runtime.capture_decoding_cuda_graph() is False       # no graphs on a CPU
    sess = runtime.open_session()
    assert sess.capabilities().max_batch_size == 2 and runtime.get_generation_metrics()["output_tokens"] == 8
    runtime.close()


def test_externalized_weights_and_refit(tmp_path):
    """Artefacts with the LM head and FFN tensors in a separate per-rank file load to the same model; refit replaces them in a
    live LLM in place, changes its outputs to the new weights' and retires cached prefixes."""
    import json
    import torch
    from tensorrt_edge_llm_b200 import AutoModel
    from tensorrt_edge_llm_b200.checkpoint import external_weights as xw
    from tensorrt_edge_llm_b200.checkpoint.artifacts import load_artifacts, write_artifacts
    from tensorrt_edge_llm_b200.checkpoint.safetensors_io import SafetensorsFile, save_file
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams

    assert xw.resolve_externalize_weights("lm_head, int4_ffn") == ["ffn", "lm_head"] and xw.resolve_externalize_weights(None) == []
    assert set(xw.resolve_externalize_weights("all")) == set(xw.EXTERNAL_WEIGHT_KINDS)
    with pytest.raises(ValueError):
        xw.resolve_externalize_weights("kv")
    assert xw.kind_of("lm_head.weight") == "lm_head" and xw.kind_of("model.layers.3.mlp.down_proj.weight") == "ffn"
    assert xw.kind_of("model.layers.0.mlp.experts.w13") == "moe" and xw.kind_of("model.embed_tokens.weight") == "embedding"
    assert xw.kind_of("model.layers.0.self_attn.qkv_proj.weight") is None

    def checkpoint(seed, d):
        cfg = tiny_llama_config(num_hidden_layers=2, dtype="float32")
        m = AutoModel.from_config(cfg, random_init=seed)
        d.mkdir()
        hf = {"model_type": "llama", "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size, "num_hidden_layers": 2,
              "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads, "vocab_size": cfg.vocab_size,
              "head_dim": cfg.head_dim, "max_position_embeddings": cfg.max_position_embeddings, "rms_norm_eps": cfg.rms_norm_eps,
              "rope_theta": cfg.rope_theta, "torch_dtype": "float32", "tie_word_embeddings": False}
        (d / "config.json").write_text(json.dumps(hf))
        state = {}
        for k, v in m.state_dict().items():               # back to Hugging Face names: split the fused projections
            if k.endswith("qkv_proj.weight"):
                q, kv = cfg.q_size, cfg.kv_size
                for name, part in zip(("q_proj", "k_proj", "v_proj"), v.split([q, kv, kv], 0)):
                    state[k.replace("qkv_proj", name)] = part.contiguous()
            elif k.endswith("gate_up_proj.weight"):
                for name, part in zip(("gate_proj", "up_proj"), v.chunk(2, 0)):
                    state[k.replace("gate_up_proj", name)] = part.contiguous()
            else:
                state[k] = v
        save_file(state, str(d / "model.safetensors"))
        return str(d)

    src_a, src_b = checkpoint(1, tmp_path / "a"), checkpoint(2, tmp_path / "b")
    world = write_artifacts(src_a, str(tmp_path / "ea"), externalize_weights="lm_head,ffn")
    write_artifacts(src_b, str(tmp_path / "eb"), externalize_weights=["lm_head", "ffn"])
    ext = world["ranks"][0]["external"]
    names = set(SafetensorsFile(str(tmp_path / "ea" / ext["weights"])).keys())
    assert ext["kinds"] == ["ffn", "lm_head"] and "lm_head.weight" in names and all(xw.kind_of(n) in ("ffn", "lm_head") for n in names)
    assert not (names & set(SafetensorsFile(str(tmp_path / "ea" / "rank0.safetensors")).keys()))
    model_a = load_artifacts(str(tmp_path / "ea"), verify=True)
    ref_a = AutoModel.from_pretrained(src_a)
    for (k, v), (_, w) in zip(model_a.state_dict().items(), ref_a.state_dict().items()):
        assert torch.equal(v, w), k
    # the external file of another preparation, read from its directory
    mixed = load_artifacts(str(tmp_path / "ea"), external_dir=str(tmp_path / "eb"))
    ref_b = AutoModel.from_pretrained(src_b)
    assert torch.equal(mixed.lm_head.weight, ref_b.lm_head.weight) and torch.equal(mixed.model.embed_tokens.weight, ref_a.model.embed_tokens.weight)
    (tmp_path / "ea" / ext["weights"]).rename(tmp_path / "ea" / "moved.safetensors")
    with pytest.raises(FileNotFoundError):
        load_artifacts(str(tmp_path / "ea"))
    (tmp_path / "ea" / "moved.safetensors").rename(tmp_path / "ea" / ext["weights"])

    # refit a live LLM: outputs follow the new weights, addresses stay, the prefix cache starts a new generation
    llm = LLM(str(tmp_path / "ea"), device="cpu", max_batch_size=2, max_input_len=128, max_kv_cache_capacity=192,
              enable_in_flight_batching=True, enable_prefix_cache=True, page_size=16)
    prompt = list(range(3, 40))
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    before = llm.generate([prompt], sp)[0].token_ids
    ptr = llm.model.lm_head.weight.data_ptr()
    stats = llm.refit(str(tmp_path / "eb" / ext["weights"]))
    assert stats["tensors"] == len(names) and stats["kinds"] == ["ffn", "lm_head"] and llm.model.lm_head.weight.data_ptr() == ptr
    reused0 = llm.engine.metrics().prefix_reused_tokens
    after = llm.generate([prompt], sp)[0].token_ids
    assert llm.engine.metrics().prefix_reused_tokens == reused0           # nothing cached under the old weights was adopted
    kv = KVCacheManager(mixed.cfg, num_pages=16, page_size=16, max_seats=1, max_pages_per_seq=12)
    runner = ModelRunner(mixed, kv)
    first = runner.prefill([0], [prompt]).argmax(-1)
    want = [int(first[0])] + runner.decode_greedy([0], first, 4)[0].tolist()
    assert after == want and after != before
    again = llm.generate([prompt], sp)[0].token_ids                        # the new generation is cached and reused
    assert again == after and llm.engine.metrics().prefix_reused_tokens > reused0
    with pytest.raises(KeyError):
        llm.refit({"no.such.tensor": torch.zeros(1)})
    with pytest.raises(ValueError):
        llm.refit({"lm_head.weight": torch.zeros(3, 3)})
    assert llm.generate([prompt], sp)[0].token_ids == after                # a refused refit changed nothing
    llm.close()


def test_stream_command_prints_pieces_as_they_are_generated(ckpt, tmp_path, capsys):
    """``trtedge stream``: a request file through the native façade; the streamed pieces concatenate to what ``infer``'s path
    (the Python generate call) produces for the same greedy requests."""
    import shutil
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    from tensorrt_edge_llm_b200.runtime import native as rt
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams
    d = str(tmp_path / "m")
    shutil.copytree(ckpt, d)
    tok = Tokenizer(models.BPE())
    pat = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=500, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(["the quick brown fox jumps over the lazy dog " * 4, "hello world how are you today"] * 3, trainer)
    tok.save(os.path.join(d, "tokenizer.json"))
    with open(os.path.join(d, "tokenizer_config.json"), "w") as f:
        json.dump({"eos_token": "<|im_end|>", "chat_template": "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}"}, f)
    body = {"temperature": 0.0, "max_generate_length": 6, "requests": [{"messages": [{"role": "user", "content": "hello world"}]},
                                                                       {"messages": [{"role": "user", "content": "the lazy dog"}]}]}
    req_file = str(tmp_path / "req.json")
    with open(req_file, "w") as f:
        json.dump(body, f)
    capsys.readouterr()
    assert trtedge(["stream", d, "--input-file", req_file, "--device", "cpu", "--max-kv-cache-capacity", "256", "--max-input-len", "128"]) == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines()]
    texts, toks = {0: "", 1: ""}, {0: [], 1: []}
    for ev in lines:
        if not ev.get("finished"):
            texts[ev["request"]] += ev["text"]
            toks[ev["request"]] += ev["tokens"]
    done = [ev for ev in lines if ev.get("finished")]
    assert len(done) == 2 and all(ev["generated_tokens"] == len(toks[ev["request"]]) and ev["error"] == "" for ev in done)
    # the same prompts through the Python generate call
    ntok = rt.Tokenizer.load_from_hf(d)
    from tensorrt_edge_llm_b200.chat_template import ChatTemplate
    tpl = ChatTemplate.load(d)
    prompts = [list(ntok.encode(tpl.apply(r["messages"], True, enable_thinking=False))) for r in body["requests"]]
    llm = LLM(d, device="cpu", max_batch_size=2, max_input_len=128, max_kv_cache_capacity=256)
    want = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=6))]
    llm.close()
    assert [toks[0], toks[1]] == want
    assert texts[0] == ntok.decode(want[0], True).decode("utf-8", "replace")
    # --plain needs exactly one request
    assert trtedge(["stream", d, "--input-file", req_file, "--plain", "--device", "cpu"]) == 2


def test_awq_search_lowers_the_output_error_of_int4_rounding(tmp_path):
    """Activation-aware scaling on a checkpoint whose activations have a few dominant channels: the searched
    ``pre_quant_scale`` is shared by fused projections, differs from 1, and the quantised model's logits are closer to the
    16-bit model's than with plain rounding."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from tensorrt_edge_llm_b200.quantization.quantize import awq_search, quantize_and_export
    d = str(tmp_path / "m")
    os.makedirs(d)
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=32, rms_norm_eps=1e-6, rope_theta=1e4, max_position_embeddings=256, tie_word_embeddings=False)
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg).float().eval()
    with torch.no_grad():                                   # a few loud input channels: norm weights with outliers
        for layer in m.model.layers:
            layer.input_layernorm.weight[:6] = 12.0
            layer.post_attention_layernorm.weight[10:14] = 9.0
    save_file(dict(m.state_dict()), os.path.join(d, "model.safetensors"))
    hf = cfg.to_dict()
    hf["torch_dtype"] = "float32"
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    pqs = awq_search(d, group_size=64)
    q, k, g, u = (pqs.get(f"model.layers.0.{n}") for n in ("self_attn.q_proj", "self_attn.k_proj", "mlp.gate_proj", "mlp.up_proj"))
    assert q is not None and torch.equal(q, k) and g is not None and torch.equal(g, u)           # fused projections share a scale
    assert float((q - 1).abs().max()) > 0.05 and q[:6].mean() < q[6:].mean()                      # loud channels are scaled up in W
    ids = list(range(5, 60))
    ref_logits = _logits(d, ids)
    errs = {}
    for calibrate in (False, True):
        out = str(tmp_path / f"q{int(calibrate)}")
        quantize_and_export(d, out, "int4_awq", calibrate=calibrate, group_size=64)
        f = SafetensorsFile(os.path.join(out, "model.safetensors"))
        assert ("model.layers.0.self_attn.q_proj.pre_quant_scale" in set(f.keys())) == calibrate
        errs[calibrate] = float((_logits(out, ids) - ref_logits).pow(2).mean())
    assert errs[True] < errs[False]


def test_gptq_error_compensation_beats_plain_rounding(ckpt, tmp_path):
    """GPTQ on correlated inputs: the layer's output error is well below round-to-nearest with the same group layout, the
    export decodes to the compensated weights, and the quantised checkpoint loads."""
    from tensorrt_edge_llm_b200.checkpoint import repacking as rp
    from tensorrt_edge_llm_b200.quantization.quantize import gptq_quantize, quantize_and_export
    g = torch.Generator().manual_seed(0)
    n_in, n_out, group = 128, 48, 32
    basis = torch.randn(8, n_in, generator=g)
    x = torch.randn(400, 8, generator=g) @ basis + 0.05 * torch.randn(400, n_in, generator=g)      # low-rank, strongly correlated
    w = torch.randn(n_out, n_in, generator=g)
    codes, sc, zp = gptq_quantize(w, x, group, block=64)
    assert codes.min() >= 0 and codes.max() <= 15 and sc.shape == (n_out, n_in // group)
    w_gptq = (codes - zp.repeat_interleave(group, 1)) * sc.repeat_interleave(group, 1)
    w_rtn = rp.decode_gptq(**rp.encode_gptq(w, group))
    err = lambda wq: float((x @ (wq - w).t()).pow(2).mean())
    assert err(w_gptq) < 0.5 * err(w_rtn)
    out = str(tmp_path / "gq")
    quantize_and_export(ckpt, out, "int4_gptq", group_size=64)
    f = SafetensorsFile(os.path.join(out, "model.safetensors"))
    assert f.info("model.layers.0.mlp.down_proj.qweight")[1] == [256 // 8, 128]
    ids = list(range(5, 45))
    a, b = _logits(ckpt, ids), _logits(out, ids)
    assert float(torch.nn.functional.cosine_similarity(a - a.mean(), b - b.mean(), dim=-1)) > 0.97
