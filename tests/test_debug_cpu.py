"""Layer dumps and teacher forcing through environment variables."""
import json
import os

import torch

from tensorrt_edge_llm_b200.checkpoint.safetensors_io import SafetensorsFile
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.llm import LLM
from tensorrt_edge_llm_b200.runtime.runner import SamplingParams


def test_layer_dump_and_teacher_forcing(tmp_path, monkeypatch):
    cfg = tiny_llama_config(num_hidden_layers=3, dtype="float32")
    prompts = [[5, 6, 7, 8], [9, 10, 11]]
    plain = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=64, max_kv_cache_capacity=96, page_size=16)
    free_run = plain.generate(prompts, SamplingParams(max_tokens=4, ignore_eos=True))
    forced = [[1, 2, 3, 4], [4, 3, 2, 1]]
    (tmp_path / "force.json").write_text(json.dumps(forced))
    monkeypatch.setenv("TELB_DUMP_LAYERS_DIR", str(tmp_path / "dump"))
    monkeypatch.setenv("TELB_DUMP_LAYERS", "0,2")
    monkeypatch.setenv("TELB_FORCE_TOKENS_FILE", str(tmp_path / "force.json"))
    dbg = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=64, max_kv_cache_capacity=96, page_size=16)
    outs = dbg.generate(prompts, SamplingParams(max_tokens=4, ignore_eos=True))
    assert [o.token_ids for o in outs] == forced and [o.token_ids for o in free_run] != forced
    files = sorted(os.listdir(tmp_path / "dump"))
    assert files == ["step0.safetensors", "step1.safetensors", "step2.safetensors", "step3.safetensors"]      # prefill + 3 forced steps
    f0 = SafetensorsFile(str(tmp_path / "dump" / "step0.safetensors"))
    assert sorted(f0.keys()) == ["layer0.hidden", "layer2.hidden", "logits"]
    assert f0.info("layer0.hidden")[1] == [7, cfg.hidden_size] and f0.info("logits")[1] == [2, cfg.vocab_size]
    # the dumped prefill logits are the ones the plain run sampled its first token from
    assert f0.get("logits").argmax(-1).tolist() == [o.token_ids[0] for o in free_run]
    f1 = SafetensorsFile(str(tmp_path / "dump" / "step1.safetensors"))
    assert f1.info("layer2.hidden")[1] == [2, cfg.hidden_size]
