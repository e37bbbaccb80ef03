"""``trtedge build <checkpoint> --output_dir …``: validate a checkpoint and write the runtime artefacts.

The reference compiles TensorRT engines here (``tensorrt_edgellm/builder/``, ``cpp/builder/llmBuilder.cpp``).
This runtime executes checkpoints directly, so "build" prepares the weights once: it checks that every tensor the model
needs is present and shaped for the requested tensor-parallel degree, expands / repacks / fuses / slices them per rank and
writes the artefact set of ``checkpoint/artifacts.py`` (``world_config.json``, ``runtime_config.json``, one
``rank<r>.safetensors`` per rank, the tokenizer and config side files) — the counterpart of
``build_runtime_llm_config_dict`` and the engine directory of ``tensorrt_edgellm/checkpoint/checkpoint_utils.py:578``.
``AutoModel.from_pretrained`` / ``LLM`` / ``trtedge serve`` take that directory in place of the checkpoint.
``--config-only`` keeps the earlier behaviour (validation + ``runtime_config.json`` beside the checkpoint)."""
import argparse
import json
import os
import sys

from ..checkpoint.artifacts import runtime_config_dict, write_artifacts     # noqa: F401  (runtime_config_dict is re-exported)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge build")
    p.add_argument("model_dir")
    p.add_argument("--output_dir", "--output-dir", default="")
    p.add_argument("--max-batch-size", type=int, default=1)
    p.add_argument("--max-input-len", type=int, default=4096)
    p.add_argument("--max-kv-cache-capacity", type=int, default=8192)
    p.add_argument("--tensor-parallel-size", type=int, default=1)
    p.add_argument("--expert-parallel", action="store_true", help="shard experts by id over the ranks (MoE checkpoints)")
    p.add_argument("--externalize-weights", "--externalize_weights", default="",
                   help="comma-separated kinds kept in a separate per-rank file: lm_head, ffn, moe, embedding, all")
    p.add_argument("--config-only", action="store_true", help="validate and write runtime_config.json only, no prepared weights")
    a = p.parse_args(argv)
    import torch
    from ..checkpoint.loader import load_weights
    from ..config import Mapping, ModelConfig
    from ..model import model_class_for
    out_dir = a.output_dir or a.model_dir
    if not a.config_only and os.path.abspath(out_dir) != os.path.abspath(a.model_dir):
        try:
            world = write_artifacts(a.model_dir, out_dir, a.tensor_parallel_size, a.max_batch_size, a.max_input_len,
                                    a.max_kv_cache_capacity, a.expert_parallel, a.externalize_weights or None)
        except KeyError as e:
            print(json.dumps({"ok": False, "missing": [str(e)]}))
            return 1
        except ValueError as e:
            print(json.dumps({"ok": False, "error": str(e)}))
            return 2
        print(json.dumps({"ok": True, "runtime_config": os.path.join(out_dir, "runtime_config.json"),
                          "world_config": os.path.join(out_dir, "world_config.json"),
                          "weights": [r["weights"] for r in world["ranks"]], "bytes": sum(r["bytes"] for r in world["ranks"]),
                          "external_weights": [r["external"]["weights"] for r in world["ranks"] if "external" in r]}))
        return 0
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
    os.makedirs(out_dir, exist_ok=True)
    cfg = ModelConfig.from_pretrained(a.model_dir)
    with open(os.path.join(out_dir, "runtime_config.json"), "w", encoding="utf-8") as f:
        json.dump(runtime_config_dict(cfg, a.max_batch_size, a.max_input_len, a.max_kv_cache_capacity, a.tensor_parallel_size), f,
                  indent=1, default=str)
    print(json.dumps({"ok": True, "runtime_config": os.path.join(out_dir, "runtime_config.json")}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
