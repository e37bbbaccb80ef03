"""``trtedge build <checkpoint> --output_dir …``: validate a checkpoint and write the runtime artifacts.

The reference compiles TensorRT engines here (``tensorrt_edgellm/builder/``, ``cpp/builder/llmBuilder.cpp``).
This runtime executes checkpoints directly, so "build" checks that every tensor the model needs is present
and shaped for the requested tensor-parallel degree, and writes ``runtime_config.json`` (the parsed model,
quantisation and deployment limits — the counterpart of ``build_runtime_llm_config_dict``,
``tensorrt_edgellm/checkpoint/checkpoint_utils.py:578``)."""
import argparse
import dataclasses
import json
import os
import sys


def runtime_config_dict(cfg, max_batch_size: int, max_input_len: int, max_kv_cache_capacity: int, tp: int) -> dict:
    d = dataclasses.asdict(cfg)
    d.pop("mapping", None)
    return {"model": d, "deployment": {"max_batch_size": max_batch_size, "max_input_len": max_input_len,
                                       "max_kv_cache_capacity": max_kv_cache_capacity, "tensor_parallel_size": tp, "kv_page_size": 64},
            "format": "tensorrt_edge_llm_b200.runtime_config.v1"}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge build")
    p.add_argument("model_dir")
    p.add_argument("--output_dir", "--output-dir", default="")
    p.add_argument("--max-batch-size", type=int, default=1)
    p.add_argument("--max-input-len", type=int, default=4096)
    p.add_argument("--max-kv-cache-capacity", type=int, default=8192)
    p.add_argument("--tensor-parallel-size", type=int, default=1)
    a = p.parse_args(argv)
    import torch
    from ..checkpoint.loader import load_weights
    from ..config import Mapping, ModelConfig
    from ..model import model_class_for
    missing = []
    for rank in range(a.tensor_parallel_size):
        cfg = ModelConfig.from_pretrained(a.model_dir, Mapping(tp_size=a.tensor_parallel_size, tp_rank=rank))
        with torch.device("meta"):
            model = model_class_for(cfg)(cfg, None)
        model = model.to_empty(device="cpu")
        try:
            load_weights(model, a.model_dir, strict=True)
        except KeyError as e:
            missing.append(f"rank {rank}: {e}")
    if missing:
        print(json.dumps({"ok": False, "missing": missing}))
        return 1
    out_dir = a.output_dir or a.model_dir
    os.makedirs(out_dir, exist_ok=True)
    cfg = ModelConfig.from_pretrained(a.model_dir)
    with open(os.path.join(out_dir, "runtime_config.json"), "w", encoding="utf-8") as f:
        json.dump(runtime_config_dict(cfg, a.max_batch_size, a.max_input_len, a.max_kv_cache_capacity, a.tensor_parallel_size), f,
                  indent=1, default=str)
    print(json.dumps({"ok": True, "runtime_config": os.path.join(out_dir, "runtime_config.json")}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
