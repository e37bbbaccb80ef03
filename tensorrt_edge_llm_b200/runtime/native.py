"""Loader of the native runtime module (``_lib/_telb_runtime*.so``).

``from tensorrt_edge_llm_b200.runtime import native as rt`` then ``rt.RequestEngine`` etc.
Parity: the lazy façade ``tensorrt_edgellm/runtime.py`` over ``_edgellm_runtime`` in the reference.
"""
from __future__ import annotations

import glob
import importlib.util
import os
import sys

_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_lib")


def _load():
    cands = sorted(glob.glob(os.path.join(_DIR, "_telb_runtime*.so")))
    if not cands:
        raise ImportError(f"native runtime not built under {_DIR}: run `python -m tensorrt_edge_llm_b200.build`")
    spec = importlib.util.spec_from_file_location("_telb_runtime", cands[-1])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules.setdefault("_telb_runtime", mod)
    return mod


_mod = _load()
globals().update({k: getattr(_mod, k) for k in dir(_mod) if not k.startswith("__")})
