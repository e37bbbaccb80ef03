"""B200-native Edge-LLM runtime.

Public surface (same names as ``tensorrt_edgellm/__init__.py:28-37`` of the reference):
``AutoModel, ModelConfig, QuantConfig, export_onnx, load_checkpoint_config_dicts,
load_config_dict, load_weights, register_model``.
"""
from ._version import __version__
from .config import (Mapping, ModelConfig, QuantConfig, MambaConfig, GdnConfig, load_checkpoint_config_dicts,
                     load_config_dict)
from .model import AutoModel, register_model


def load_weights(model, model_dir, strict=True):
    from .checkpoint.loader import load_weights as _lw
    return _lw(model, model_dir, strict)


def export_onnx(model, path, *a, **kw):
    """Optional interoperability dump; the execution path never needs ONNX."""
    from .utils.export import export_onnx as _e
    return _e(model, path, *a, **kw)


__all__ = ["__version__", "AutoModel", "ModelConfig", "QuantConfig", "Mapping", "MambaConfig", "GdnConfig",
           "export_onnx", "load_checkpoint_config_dicts", "load_config_dict", "load_weights", "register_model"]
