from __future__ import annotations

import json
import os
import re
import shutil
from typing import Dict, List, Tuple

import torch

from ..checkpoint.safetensors_io import CheckpointReader, save_file

_KEY = re.compile(r"^(?:base_model\.model\.)?(?P<mod>.+?)\.lora_(?P<ab>[AB])(?:\.default)?\.weight$")


def _adapter(adapter_dir: str) -> Tuple[Dict[str, Dict[str, torch.Tensor]], float, int]:
    with open(os.path.join(adapter_dir, "adapter_config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    r, alpha = int(cfg["r"]), float(cfg.get("lora_alpha", cfg["r"]))
    path = os.path.join(adapter_dir, "adapter_model.safetensors")
    reader = CheckpointReader(adapter_dir) if not os.path.exists(path) else None
    from ..checkpoint.safetensors_io import SafetensorsFile
    src = SafetensorsFile(path) if reader is None else reader
    mods: Dict[str, Dict[str, torch.Tensor]] = {}
    for k in src.keys():
        m = _KEY.match(k)
        if m:
            mods.setdefault(m.group("mod"), {})[m.group("ab")] = src.get(k).clone()
    return mods, alpha / r, r


def lora_target_modules(adapter_dir: str) -> List[str]:
    """Checkpoint module names the adapter touches (where the runtime binds ``lora_A_*`` / ``lora_B_*``)."""
    return sorted(_adapter(adapter_dir)[0])


def process_lora_weights(adapter_dir: str, out_dir: str, dtype: torch.dtype = torch.float16) -> dict:
    """PEFT adapter → runtime adapter file: ``lora_A_<module> [r, in]``, ``lora_B_<module> [out, r]`` with the
    ``alpha / r`` scale folded into B, plus ``lora_config.json`` (rank, modules)."""
    mods, scale, r = _adapter(adapter_dir)
    out = {}
    for mod, ab in mods.items():
        if "A" not in ab or "B" not in ab:
            raise ValueError(f"adapter module {mod} lacks lora_A or lora_B")
        out[f"lora_A_{mod}"] = ab["A"].to(dtype).contiguous()
        out[f"lora_B_{mod}"] = (ab["B"].float() * scale).to(dtype).contiguous()
    os.makedirs(out_dir, exist_ok=True)
    save_file(out, os.path.join(out_dir, "lora_weights.safetensors"))
    meta = {"rank": r, "scale_folded_into_B": True, "modules": sorted(mods)}
    with open(os.path.join(out_dir, "lora_config.json"), "w", encoding="utf-8") as f:
        json.dump(meta, f, indent=1)
    return meta


def merge_lora(model_dir: str, adapter_dir: str, out_dir: str) -> dict:
    """``W ← W + (alpha / r) · B A`` for every adapted module of a 16-bit checkpoint."""
    mods, scale, _ = _adapter(adapter_dir)
    reader = CheckpointReader(model_dir)
    out, merged = {}, 0
    for key in reader.keys():
        t = reader.get(key)
        mod = key[:-len(".weight")] if key.endswith(".weight") else None
        ab = mods.get(mod) if mod else None
        if ab is None and mod and mod.startswith("model."):
            ab = mods.get(mod[len("model."):])
        if ab is not None:
            if t.dtype not in (torch.float16, torch.bfloat16, torch.float32):
                raise ValueError(f"{key}: merging needs a 16-bit or fp32 base weight, found {t.dtype}")
            out[key] = (t.float() + scale * (ab["B"].float() @ ab["A"].float())).to(t.dtype)
            merged += 1
        else:
            out[key] = t.clone()
    os.makedirs(out_dir, exist_ok=True)
    save_file(out, os.path.join(out_dir, "model.safetensors"))
    for fname in os.listdir(model_dir):
        if fname.endswith((".json", ".jinja", ".txt", ".model")) and not fname.startswith("model.safetensors"):
            shutil.copy(os.path.join(model_dir, fname), os.path.join(out_dir, fname))
    if merged != len(mods):
        raise ValueError(f"adapter has {len(mods)} modules but only {merged} matched checkpoint weights")
    return {"merged_modules": merged}
