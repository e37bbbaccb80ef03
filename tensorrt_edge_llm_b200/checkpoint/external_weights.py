"""Externalised weights and refit.

Part of a prepared model can live outside the rank's main weight file: the LM head, the dense FFN projections, the expert
tensors, the embedding table — the large blocks that a deployment may want to keep on a different medium, share between
variants of one model, or replace without preparing the whole model again.  ``write_artifacts(..., externalize_weights=[...])``
puts the tensors of the chosen kinds into ``rank<r>.external.safetensors`` and records them in the world configuration;
``load_artifacts`` reads both files (the external one optionally from another directory).

``refit`` replaces tensors of a live model in place from such a file (or from any safetensors file or dict with the same
names).  Addresses do not change, so captured CUDA graphs and cached tensor maps stay valid; what does become stale is
every cached K/V row, which ``LLM.refit`` discards (it waits for the engine to drain, copies, and starts a new prefix-cache
generation).

Parity: ``tensorrt_edgellm/external_weights.py`` (kinds :24-40, ``resolve_externalize_weights`` :54, manifest :76,
``reject_quantized_lm_head_externalization`` :90) and the runtime's refit / external weight reader
(``cpp/runtime/features``); there the tensors leave an ONNX graph, here they leave the rank's prepared state."""
from __future__ import annotations

import re
from typing import Dict, Iterable, List, Optional, Sequence, Union

import torch

EXTERNAL_WEIGHT_LM_HEAD = "lm_head"
EXTERNAL_WEIGHT_FFN = "ffn"
EXTERNAL_WEIGHT_MOE = "moe"
EXTERNAL_WEIGHT_EMBEDDING = "embedding"
EXTERNAL_WEIGHT_ALL = "all"
EXTERNAL_WEIGHT_KINDS = (EXTERNAL_WEIGHT_LM_HEAD, EXTERNAL_WEIGHT_FFN, EXTERNAL_WEIGHT_MOE, EXTERNAL_WEIGHT_EMBEDDING)
# names the reference uses for the same blocks
_ALIASES = {"int4_ffn": EXTERNAL_WEIGHT_FFN, "int4_moe": EXTERNAL_WEIGHT_MOE, "nvfp4_moe": EXTERNAL_WEIGHT_MOE}

_PATTERNS = {
    EXTERNAL_WEIGHT_LM_HEAD: re.compile(r"(^|\.)lm_head\."),
    EXTERNAL_WEIGHT_MOE: re.compile(r"\.(experts|expert_fc1|expert_fc2|w13|w2)(\.|_|$)|\.mlp\.experts"),
    EXTERNAL_WEIGHT_FFN: re.compile(r"\.mlp\.(gate_up_proj|gate_proj|up_proj|down_proj)\."),
    EXTERNAL_WEIGHT_EMBEDDING: re.compile(r"(^|\.)embed_tokens\."),
}


def resolve_externalize_weights(kinds: Union[None, str, Iterable[str]]) -> List[str]:
    """Normalise a request (``None``, a comma-separated string or a list; ``all`` expands) to a sorted list of kinds."""
    if kinds is None:
        return []
    values = [v.strip() for v in kinds.split(",")] if isinstance(kinds, str) else [str(v).strip() for v in kinds]
    out = set()
    for v in values:
        if not v:
            continue
        v = _ALIASES.get(v, v)
        if v == EXTERNAL_WEIGHT_ALL:
            out.update(EXTERNAL_WEIGHT_KINDS)
        elif v in EXTERNAL_WEIGHT_KINDS:
            out.add(v)
        else:
            raise ValueError(f"unknown external weight kind {v!r}; choose from {', '.join(EXTERNAL_WEIGHT_KINDS + (EXTERNAL_WEIGHT_ALL,))}")
    return sorted(out)


def kind_of(name: str) -> Optional[str]:
    """The external-weight kind a state tensor belongs to, or None.  Expert tensors count as ``moe`` even where their module
    path also looks like an FFN projection."""
    for kind in (EXTERNAL_WEIGHT_LM_HEAD, EXTERNAL_WEIGHT_MOE, EXTERNAL_WEIGHT_FFN, EXTERNAL_WEIGHT_EMBEDDING):
        if _PATTERNS[kind].search(name):
            return kind
    return None


def split_state(state: Dict[str, torch.Tensor], kinds: Sequence[str]):
    """``(resident, external)``: the tensors that stay in the rank's main file and those of the requested kinds."""
    kinds = set(kinds)
    resident, external = {}, {}
    for name, t in state.items():
        (external if kind_of(name) in kinds else resident)[name] = t
    return resident, external


def refit(model: torch.nn.Module, source, names: Optional[Sequence[str]] = None, allow_partial: bool = True) -> dict:
    """Copy tensors from ``source`` (a safetensors path or a ``name → tensor`` dict, named as the model's state) into the live
    model in place.  Every source tensor must exist in the model with the same shape and element size; with
    ``allow_partial=False`` the source must cover the whole state.  Returns ``{"tensors": n, "bytes": b, "kinds": [...]}``."""
    if isinstance(source, str):
        from .safetensors_io import SafetensorsFile
        f = SafetensorsFile(source)
        source = {k: f.get(k) for k in f.keys()}
    if names is not None:
        wanted = set(names)
        unknown = wanted - set(source)
        if unknown:
            raise KeyError(f"refit: the source holds no tensor named {sorted(unknown)[:5]}")
        source = {k: v for k, v in source.items() if k in wanted}
    own = model.state_dict()
    unknown = sorted(set(source) - set(own))
    if unknown:
        raise KeyError(f"refit: the model has no tensor named {unknown[:5]}")
    if not allow_partial and set(own) - set(source):
        raise KeyError(f"refit: the source lacks {sorted(set(own) - set(source))[:5]}")
    plan = []
    for k, src in source.items():           # validate everything before the first byte moves
        dst = own[k]
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"refit: tensor {k} has shape {tuple(src.shape)}, the model holds {tuple(dst.shape)}")
        if src.dtype != dst.dtype and src.element_size() != dst.element_size():
            raise ValueError(f"refit: tensor {k} is {src.dtype}, the model holds {dst.dtype}")
        plan.append((dst, src.view(dst.dtype) if src.dtype != dst.dtype and not (src.dtype.is_floating_point and dst.dtype.is_floating_point) else src))
    moved = 0
    with torch.no_grad():
        for dst, src in plan:
            dst.copy_(src)
            moved += dst.numel() * dst.element_size()
    if hasattr(model, "weights_refitted"):
        model.weights_refitted()             # a model that caches derived forms of its weights rebuilds them here
    return {"tensors": len(plan), "bytes": moved, "kinds": sorted({k for k in (kind_of(n) for n in source) if k})}
