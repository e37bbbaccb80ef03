"""Runtime artefacts ("engine directory"): a checkpoint prepared once for a deployment and loaded without repacking.

The reference compiles TensorRT engines and writes per-rank engine files plus a world configuration
(``tensorrt_edgellm/checkpoint/checkpoint_utils.py``, ``cpp/builder/``, ``cpp/runtime/llmRuntimeUtils``).  This runtime has no
engine compilation; what is worth doing once per deployment is the weight preparation: reading every shard, expanding or
repacking foreign quantisation layouts (GPTQ, AutoAWQ, FP8, ...), fusing q/k/v and gate/up, slicing for the tensor-parallel
rank.  ``write_artifacts`` runs that for every rank and stores the result as one safetensors file per rank:

    <out>/world_config.json        tensor-parallel size, per-rank weight file, byte size and SHA-256, source description
    <out>/runtime_config.json      parsed model + quantisation config and the deployment limits
    <out>/rank<r>.safetensors      the rank's module state exactly as the runtime holds it before device placement
    <out>/config.json, tokenizer files, chat template, generation config    copied so the directory is self-contained

``load_artifacts`` (used by ``AutoModel.from_pretrained`` when it meets a ``world_config.json``) rebuilds the module from the
stored config and copies the rank's tensors in: no name remapping, no repacking, no slicing ("load" as opposed to "assemble").
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
import shutil
from typing import Dict, List, Optional

import torch

from .safetensors_io import SafetensorsFile, save_file

WORLD_FORMAT = "tensorrt_edge_llm_b200.world_config.v1"
RUNTIME_FORMAT = "tensorrt_edge_llm_b200.runtime_config.v1"
_SIDE_FILES = ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "special_tokens_map.json",
               "vocab.json", "merges.txt", "chat_template.jinja", "chat_template.json", "hf_quant_config.json", "preprocessor_config.json",
               "vocab_map.safetensors", "added_tokens.json")


def is_artifact_dir(path: str) -> bool:
    return os.path.isfile(os.path.join(path, "world_config.json"))


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return h.hexdigest()


def runtime_config_dict(cfg, max_batch_size: int, max_input_len: int, max_kv_cache_capacity: int, tp: int) -> dict:
    d = dataclasses.asdict(cfg)
    d.pop("mapping", None)
    return {"model": d, "deployment": {"max_batch_size": max_batch_size, "max_input_len": max_input_len,
                                       "max_kv_cache_capacity": max_kv_cache_capacity, "tensor_parallel_size": tp, "kv_page_size": 64},
            "format": RUNTIME_FORMAT}


def write_artifacts(model_dir: str, out_dir: str, tensor_parallel_size: int = 1, max_batch_size: int = 1, max_input_len: int = 4096,
                    max_kv_cache_capacity: int = 8192, expert_parallel: bool = False, externalize_weights=None) -> dict:
    """Prepare ``model_dir`` for ``tensor_parallel_size`` ranks and write the artefact set into ``out_dir``.  Returns the world
    configuration.  Raises ``KeyError`` when the checkpoint lacks a tensor some rank needs."""
    from ..config import Mapping, ModelConfig
    from ..model import model_class_for
    from .external_weights import resolve_externalize_weights, split_state
    from .loader import load_weights
    kinds = resolve_externalize_weights(externalize_weights)
    if os.path.abspath(model_dir) == os.path.abspath(out_dir):
        raise ValueError("the artefact directory must differ from the checkpoint directory (both hold *.safetensors files)")
    os.makedirs(out_dir, exist_ok=True)
    tp = int(tensor_parallel_size)
    ranks: List[dict] = []
    for rank in range(tp):
        mapping = Mapping(tp_size=tp, tp_rank=rank, **({"ep_size": tp, "ep_rank": rank} if expert_parallel else {}))
        cfg = ModelConfig.from_pretrained(model_dir, mapping)
        model = model_class_for(cfg)(cfg, None)       # a real construction: buffers the checkpoint does not carry keep their defaults
        load_weights(model, model_dir, strict=True)
        state, external = split_state({k: v for k, v in model.state_dict().items()}, kinds)
        fn = f"rank{rank}.safetensors"
        save_file(state, os.path.join(out_dir, fn), metadata={"format": "pt", "rank": str(rank), "world": str(tp)})
        entry = {"rank": rank, "weights": fn, "bytes": os.path.getsize(os.path.join(out_dir, fn)),
                 "sha256": _sha256(os.path.join(out_dir, fn)), "tensors": len(state)}
        if external:
            xfn = f"rank{rank}.external.safetensors"
            save_file(external, os.path.join(out_dir, xfn), metadata={"format": "pt", "rank": str(rank), "world": str(tp), "kinds": ",".join(kinds)})
            entry["external"] = {"weights": xfn, "bytes": os.path.getsize(os.path.join(out_dir, xfn)), "sha256": _sha256(os.path.join(out_dir, xfn)),
                                 "tensors": len(external), "kinds": kinds}
        ranks.append(entry)
        del model, state, external
    cfg = ModelConfig.from_pretrained(model_dir)
    with open(os.path.join(out_dir, "runtime_config.json"), "w", encoding="utf-8") as f:
        json.dump(runtime_config_dict(cfg, max_batch_size, max_input_len, max_kv_cache_capacity, tp), f, indent=1, default=str)
    for name in _SIDE_FILES:
        src = os.path.join(model_dir, name)
        if os.path.isfile(src):
            shutil.copyfile(src, os.path.join(out_dir, name))
    world = {"format": WORLD_FORMAT, "tensor_parallel_size": tp, "expert_parallel": bool(expert_parallel), "ranks": ranks,
             "source": {"model_dir": os.path.abspath(model_dir), "model_type": cfg.model_type, "quantization": cfg.quant.quant_type}}
    with open(os.path.join(out_dir, "world_config.json"), "w", encoding="utf-8") as f:
        json.dump(world, f, indent=1)
    return world


def read_world_config(engine_dir: str) -> dict:
    with open(os.path.join(engine_dir, "world_config.json"), "r", encoding="utf-8") as f:
        world = json.load(f)
    if world.get("format") != WORLD_FORMAT:
        raise ValueError(f"{engine_dir}: unknown world configuration format {world.get('format')!r}")
    return world


def artifact_model_config(engine_dir: str, mapping=None):
    """The model configuration stored with the artefacts (no probing of weight files), placed on ``mapping``."""
    from ..config import Mapping, ModelConfig
    with open(os.path.join(engine_dir, "runtime_config.json"), "r", encoding="utf-8") as f:
        rc = json.load(f)
    if rc.get("format") != RUNTIME_FORMAT:
        raise ValueError(f"{engine_dir}: unknown runtime configuration format {rc.get('format')!r}")
    cfg = ModelConfig.from_dict(rc["model"])
    world = read_world_config(engine_dir)
    tp = int(world["tensor_parallel_size"])
    if mapping is None:
        if tp != 1:
            raise ValueError(f"{engine_dir} was prepared for {tp} tensor-parallel ranks: pass the rank's mapping")
        mapping = Mapping()
    if mapping.tp_size != tp:
        raise ValueError(f"{engine_dir} was prepared for tensor-parallel size {tp}, the deployment asks for {mapping.tp_size}")
    cfg.mapping = mapping
    return cfg, rc.get("deployment", {})


def load_artifacts(engine_dir: str, mapping=None, comm=None, device="cpu", verify: bool = False, external_dir: Optional[str] = None):
    """Build the rank's model from an artefact directory.  ``verify`` re-hashes the weight files against the world config;
    ``external_dir`` reads the rank's externalised tensors from another directory (same file name)."""
    from ..model import model_class_for
    cfg, _ = artifact_model_config(engine_dir, mapping)
    world = read_world_config(engine_dir)
    entry = next((r for r in world["ranks"] if int(r["rank"]) == cfg.mapping.tp_rank), None)
    if entry is None:
        raise ValueError(f"{engine_dir} holds no weights for rank {cfg.mapping.tp_rank}")
    path = os.path.join(engine_dir, entry["weights"])
    if verify and _sha256(path) != entry["sha256"]:
        raise ValueError(f"{path}: contents do not match the world configuration (sha256)")
    model = model_class_for(cfg)(cfg, comm)
    f = SafetensorsFile(path)
    state: Dict[str, torch.Tensor] = {k: f.get(k) for k in f.keys()}
    ext = entry.get("external")
    if ext:
        xpath = os.path.join(external_dir or engine_dir, ext["weights"])
        if not os.path.isfile(xpath):
            raise FileNotFoundError(f"{xpath}: the externalised weights ({', '.join(ext.get('kinds', []))}) of rank {cfg.mapping.tp_rank} are missing")
        if verify and external_dir is None and _sha256(xpath) != ext["sha256"]:
            raise ValueError(f"{xpath}: contents do not match the world configuration (sha256)")
        xf = SafetensorsFile(xpath)
        state.update({k: xf.get(k) for k in xf.keys()})
    own = model.state_dict()
    missing = sorted(set(own) - set(state))
    unexpected = sorted(set(state) - set(own))
    if missing or unexpected:
        raise KeyError(f"{path} does not fit the model: missing {missing[:5]}, unexpected {unexpected[:5]}")
    with torch.no_grad():
        for k, dst in own.items():
            src = state[k]
            if tuple(src.shape) != tuple(dst.shape):
                raise ValueError(f"{path}: tensor {k} has shape {tuple(src.shape)}, the model wants {tuple(dst.shape)}")
            dst.copy_(src.view(dst.dtype) if src.dtype != dst.dtype and src.element_size() == dst.element_size() else src)
    # the stored tensors are past `finalize_checkpoint` (it ran inside load_weights when the artefacts were written); a model
    # that keeps part of that conversion outside its tensors restores it here
    if hasattr(model, "artifacts_loaded"):
        model.artifacts_loaded()
    model.to(device).eval()
    if hasattr(model, "finalize"):
        model.finalize()
    return model
