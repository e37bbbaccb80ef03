"""Load Hugging Face / ModelOpt checkpoints into the runtime's modules.

Walks the module tree; every ``LinearBase`` pulls the tensors of the checkpoint modules it
fuses (``sources``) and shards them for its tensor-parallel rank while copying; everything
else is a name match.  Parity: ``tensorrt_edgellm/checkpoint/loader.py:145`` (``load_weights``,
``_shard_for_module``).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
from torch import nn

from ..models.linear import LinearBase, NVFP4Linear, Int4AwqLinear
from .safetensors_io import CheckpointReader

_LINEAR_FIELDS = ("weight", "weight_scale", "weight_scale_2", "input_scale", "bias", "pre_quant_scale",
                  "qweight", "qzeros", "scales", "g_idx", "weight_scale_inv")


def _strip_prefixes(keys) -> Dict[str, str]:
    """Map canonical names (``model.layers…``, ``lm_head…``) to checkpoint keys, dropping the
    wrappers multimodal checkpoints add (``language_model.``, ``model.language_model.``)."""
    out: Dict[str, str] = {}
    for k in keys:
        c = k
        for pre in ("model.language_model.", "language_model.model.", "language_model."):
            if c.startswith(pre):
                c = ("model." + c[len(pre):]) if not c[len(pre):].startswith("lm_head") else c[len(pre):]
                break
        out.setdefault(c, k)
    return out


@torch.no_grad()
def load_weights(model: nn.Module, model_dir: str, strict: bool = True) -> List[str]:
    """Fill ``model`` from the safetensors shards in ``model_dir``; returns unused checkpoint keys."""
    reader = CheckpointReader(model_dir)
    names = _strip_prefixes(reader.keys())
    remap = getattr(model, "checkpoint_key_remap", None)
    if remap is not None:       # family-specific renames (a None result drops the tensor)
        names = {remap(c): k for c, k in names.items() if remap(c) is not None}
    used = set()

    def fetch(name: str) -> Optional[torch.Tensor]:
        k = names.get(name)
        if k is None:
            return None
        used.add(k)
        return reader.get(k)

    for mod_name, mod in model.named_modules():
        if isinstance(mod, LinearBase):
            parent = mod_name.rsplit(".", 1)[0] if "." in mod_name else ""
            srcs = mod.sources or [mod_name.rsplit(".", 1)[-1]]
            bundles = []
            for s in srcs:
                base = f"{parent}.{s}" if parent else s
                b = {}
                for fld in _LINEAR_FIELDS:
                    t = fetch(f"{base}.{fld}")
                    if t is not None:
                        b[fld] = t
                if "weight_scale_inv" in b:                      # block-free FP8 exports name the scale this way
                    b.setdefault("weight_scale", b.pop("weight_scale_inv"))
                if "weight" not in b and "qweight" not in b:
                    if mod_name == "lm_head" and getattr(model, "cfg", None) is not None and model.cfg.tie_word_embeddings:
                        b["weight"] = fetch("model.embed_tokens.weight")
                    if b.get("weight") is None and "qweight" not in b:
                        if strict:
                            raise KeyError(f"checkpoint has no tensor {base}.weight")
                        b = None
                bundles.append(b)
            if all(b is not None for b in bundles):
                mod.load_from(bundles)   # type: ignore[arg-type]
    custom_prefixes = []
    for mod_name, mod in model.named_modules():
        if hasattr(mod, "load_checkpoint") and not isinstance(mod, LinearBase):
            if mod.load_checkpoint(fetch):
                custom_prefixes.append(mod_name + ".w")       # stacked expert tensors are filled by the hook
    lin_prefixes = tuple([n + "." for n, m in model.named_modules() if isinstance(m, LinearBase)] + custom_prefixes)
    for pname, p in list(model.named_parameters()) + list(model.named_buffers()):
        if pname.startswith(lin_prefixes):
            continue
        t = fetch(pname)
        if t is None:
            continue
        if t.shape != p.shape:
            t = _shard_like(t, p, model)
        p.data.copy_(t.to(p.dtype))
    if hasattr(model, "finalize_checkpoint"):
        model.finalize_checkpoint()
    reader_keys = set(reader.keys())
    return sorted(reader_keys - used)


def _shard_like(t: torch.Tensor, p: torch.Tensor, model) -> torch.Tensor:
    cfg = getattr(model, "cfg", None)
    world, rank = (cfg.tp_size, cfg.tp_rank) if cfg is not None else (1, 0)
    for d in range(t.dim()):
        if t.shape[d] == p.shape[d] * world:
            return t.narrow(d, rank * p.shape[d], p.shape[d])
    raise ValueError(f"cannot shard tensor of shape {tuple(t.shape)} into {tuple(p.shape)}")


@torch.no_grad()
def init_random_weights(model: nn.Module, seed: int = 0, std: float = 0.02) -> nn.Module:
    """N(0, std) initialisation of every weight (norm weights stay 1), quantising on the fly
    for NVFP4 / INT4 layers.  Used by the benchmarks: no checkpoint download is possible."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    for name, mod in model.named_modules():
        if isinstance(mod, (NVFP4Linear, Int4AwqLinear)):
            dev = mod.weight.device
            ws = []
            for n in mod.out_sizes:
                ws.append(_randn_chunked((n, mod.in_features), g, std, dev))
            mod.quantize_from(ws)
        elif isinstance(mod, LinearBase):
            mod.weight.data.copy_(_randn_chunked(tuple(mod.weight.shape), g, std, mod.weight.device).to(mod.weight.dtype))
        elif isinstance(mod, nn.Embedding):
            mod.weight.data.copy_(_randn_chunked(tuple(mod.weight.shape), g, std, mod.weight.device).to(mod.weight.dtype))
    for name, mod in model.named_modules():
        if hasattr(mod, "random_init") and not isinstance(mod, LinearBase):
            mod.random_init(g, std)
    return model


def _randn_chunked(shape, g, std, device) -> torch.Tensor:
    """Deterministic N(0,std): generated on CPU for small tensors (bit-stable across devices);
    large tensors are drawn on the target device from a seed derived from the CPU stream."""
    numel = 1
    for s in shape:
        numel *= s
    if device.type == "cpu" or numel <= (1 << 22):
        return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(device)
    seed = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=g))
    dg = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=dg, dtype=torch.float32, device=device) * std
