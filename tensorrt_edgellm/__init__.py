"""Drop-in import name of the reference package, backed by ``tensorrt_edge_llm_b200``.

``import tensorrt_edgellm`` and the sub-modules users reach for (``tensorrt_edgellm.server``, ``.config``,
``.model``, ``.cli``, ``.lora``, ``.quantization``, ``.vocab_reduction``, ``.chat_template``, ``.checkpoint``)
resolve to this runtime's implementations."""
import importlib
import sys

import tensorrt_edge_llm_b200 as _impl
from tensorrt_edge_llm_b200 import *  # noqa: F401,F403
from tensorrt_edge_llm_b200 import __all__, __version__  # noqa: F401

for _name in ("server", "config", "model", "cli", "lora", "quantization", "vocab_reduction", "chat_template", "checkpoint",
              "models", "runtime", "parallel", "ops"):
    _mod = importlib.import_module(f"tensorrt_edge_llm_b200.{_name}")
    sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod
