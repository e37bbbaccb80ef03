"""``trtedge insert-lora``: declare where LoRA adapters attach to a model.

In the reference this rewrites an ONNX graph so that engines expose ``lora_A_*`` / ``lora_B_*`` inputs with a maximum rank
(``tensorrt_edgellm/lora/``).  Here adapters bind to the live model, so what is worth deciding ahead of time is *which layers
are adaptable and up to which rank*: with ``--model_dir`` the command maps every module of the adapter to its runtime linear
layer (fused projections included: ``q_proj`` → columns of ``qkv_proj``), checks the factor shapes against the layer, and writes
``lora_slots.json`` beside the model.  ``LLM`` reads that file at load and wraps the listed layers before the first step, so
later ``load_lora`` calls find their slots and layers that would otherwise re-pack their weights for fused epilogues keep the
plain layout.  Without ``--model_dir`` it only lists the adapter's modules."""
import argparse
import json
import os
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge insert-lora")
    p.add_argument("--lora_dir", "--lora-dir", required=True, help="a PEFT adapter directory")
    p.add_argument("--model_dir", "--model-dir", "--onnx_dir", "--onnx-dir", default="", help="checkpoint or artefact directory to declare slots in")
    p.add_argument("--max_lora_rank", "--max-lora-rank", type=int, default=0, help="largest adapter rank to allow (default: this adapter's)")
    a = p.parse_args(argv)
    from ..lora import lora_target_modules
    from ..lora.lora import _adapter
    modules = lora_target_modules(a.lora_dir)
    if not a.model_dir:
        print(json.dumps({"modules": modules, "note": "pass --model_dir to declare adapter slots for a model"}))
        return 0
    import torch
    from ..checkpoint.artifacts import artifact_model_config, is_artifact_dir
    from ..config import ModelConfig
    from ..lora.runtime import LoraManager
    from ..model import model_class_for
    cfg = artifact_model_config(a.model_dir)[0] if is_artifact_dir(a.model_dir) else ModelConfig.from_pretrained(a.model_dir)
    with torch.device("meta"):
        model = model_class_for(cfg)(cfg, None)
    mgr = LoraManager(model)
    mods, _, rank = _adapter(a.lora_dir)
    slots, problems = {}, []
    for ckpt_mod in modules:
        try:
            mod_name, src, base = mgr._locate(ckpt_mod)
        except KeyError as e:
            problems.append(str(e))
            continue
        fa, fb = mods[ckpt_mod].get("A"), mods[ckpt_mod].get("B")
        n_in = base.in_features * (base.tp_size if getattr(base, "tp_size", 1) > 1 and str(base.tp_mode).endswith("ROW") else 1)
        n_out = base.out_sizes[src] * (base.tp_size if getattr(base, "tp_size", 1) > 1 and str(base.tp_mode).endswith("COL") else 1)
        if fa is None or fb is None:
            problems.append(f"{ckpt_mod}: lora_A or lora_B missing")
        elif tuple(fa.shape) != (rank, n_in) or tuple(fb.shape) != (n_out, rank):
            problems.append(f"{ckpt_mod}: factors {tuple(fa.shape)} / {tuple(fb.shape)} do not fit a [{n_out}, {n_in}] layer at rank {rank}")
        else:
            slots[ckpt_mod] = {"module": mod_name, "source": src, "in_features": n_in, "out_features": n_out}
    if problems:
        print(json.dumps({"ok": False, "problems": problems}))
        return 1
    max_rank = max(int(a.max_lora_rank or 0), rank)
    path = os.path.join(a.model_dir, "lora_slots.json")
    prior = {}
    if os.path.isfile(path):
        with open(path, "r", encoding="utf-8") as f:
            prior = json.load(f)
    merged = {**prior.get("slots", {}), **slots}
    out = {"max_lora_rank": max(max_rank, int(prior.get("max_lora_rank", 0))), "slots": merged}
    with open(path, "w", encoding="utf-8") as f:
        json.dump(out, f, indent=1)
    print(json.dumps({"ok": True, "lora_slots": path, "max_lora_rank": out["max_lora_rank"], "modules": sorted(merged)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
