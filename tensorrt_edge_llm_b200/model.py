"""``AutoModel`` and the model-family registry.

Parity: ``tensorrt_edgellm/model.py:289-293`` (``AutoModel.from_pretrained``,
``register_model``).  A family is a callable ``(ModelConfig, comm) -> nn.Module`` keyed by the
Hugging Face ``model_type``.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from .config import Mapping, ModelConfig

_REGISTRY: Dict[str, Callable] = {}


def register_model(*model_types: str):
    """Decorator: register a model class / factory for one or more ``model_type`` strings."""
    def deco(factory):
        for t in model_types:
            _REGISTRY[t] = factory
        return factory
    return deco


def _ensure_builtin():
    if "llama" in _REGISTRY:
        return
    from .models.default import CausalLM
    for t in ("llama", "qwen2", "qwen3", "mistral", "phi3", "gemma", "default"):
        _REGISTRY[t] = CausalLM
    from .models import qwen3_moe, nemotron_h, eagle3, eagle4, mtp, gemma, diffusion_gemma, dflash, dflash2, lilicorr, dspark, tts  # noqa: F401  (register themselves)


def model_class_for(cfg: ModelConfig):
    _ensure_builtin()
    if cfg.draft_type == "eagle3":
        return _REGISTRY["eagle4" if cfg.is_eagle4_draft else "eagle3"]
    if cfg.draft_type == "dflash":
        if cfg.dflash_version == 2:
            return _REGISTRY["lilicorr" if cfg.dflash_projector_type == "lilicorr" else "dflash2"]
        if cfg.dflash_projector_type == "dspark":
            return _REGISTRY["dspark"]
        return _REGISTRY["domino" if cfg.dflash_projector_type == "domino" else "dflash"]
    if cfg.draft_type == "mtp":
        return _REGISTRY["mtp"]
    if cfg.model_type in _REGISTRY:
        return _REGISTRY[cfg.model_type]
    if cfg.is_hybrid:
        return _REGISTRY["nemotron_h_hybrid"]
    if cfg.is_moe:
        return _REGISTRY["qwen3_moe"]
    return _REGISTRY["default"]


class AutoModel:
    """Build a runnable model from a checkpoint directory or from a config with random weights."""

    @staticmethod
    def from_config(cfg: ModelConfig, comm=None, device="cpu", random_init: Optional[int] = None):
        cls = model_class_for(cfg)
        with torch.device(device):
            model = cls(cfg, comm)
        if random_init is not None:
            from .checkpoint.loader import init_random_weights
            init_random_weights(model, seed=random_init)
        model.eval()
        if hasattr(model, "finalize"):
            model.finalize()
        return model

    @staticmethod
    def from_pretrained(model_dir: str, mapping: Optional[Mapping] = None, comm=None, device="cpu"):
        from .checkpoint.artifacts import is_artifact_dir, load_artifacts
        from .checkpoint.loader import load_weights
        if is_artifact_dir(model_dir):          # prepared by `trtedge build`: load the rank's tensors as stored
            return load_artifacts(model_dir, mapping, comm, device)
        cfg = ModelConfig.from_pretrained(model_dir, mapping)
        cls = model_class_for(cfg)
        model = cls(cfg, comm)
        load_weights(model, model_dir)
        model.to(device).eval()
        if hasattr(model, "finalize"):
            model.finalize()
        return model
