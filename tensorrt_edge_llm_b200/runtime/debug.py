"""Debug aids driven by environment variables: per-layer hidden-state dumps and teacher forcing.

``TELB_DUMP_LAYERS_DIR=<dir>`` (optionally ``TELB_DUMP_LAYERS=0,5,35``): every forward pass writes the residual
stream after the selected decoder layers, and the final logits, to ``<dir>/step<k>.safetensors`` — the files a
golden comparison against a Hugging Face run needs.  ``TELB_FORCE_TOKENS_FILE=<json>``: the static-batch generator
feeds the listed token ids (``[[...], [...]]``, one list per sequence) instead of its own samples, so logits can be
compared position by position even after the first divergence.

Parity: ``cpp/runtime/debug/layerDebugger*`` (``EDGELLM_DUMP_LOGITS_KVCACHE_LAYERS`` / ``_DIR``,
``EDGELLM_FORCE_TOKENS_FILE``) and the few-layer validation flow of ``tests/compare_layer_dumps.py``."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch


class LayerDumper:
    def __init__(self, out_dir: str, layers: Optional[List[int]] = None):
        self.out_dir, self.layers, self.step = out_dir, layers, 0
        os.makedirs(out_dir, exist_ok=True)
        self._handles = []
        self._cur: Dict[str, torch.Tensor] = {}

    @classmethod
    def from_env(cls) -> Optional["LayerDumper"]:
        d = os.environ.get("TELB_DUMP_LAYERS_DIR")
        if not d:
            return None
        sel = os.environ.get("TELB_DUMP_LAYERS")
        return cls(d, [int(x) for x in sel.split(",")] if sel else None)

    def attach(self, model) -> "LayerDumper":
        """Hook the decoder layers (their outputs are ``(block output, residual stream)``) and the model's logits."""
        for i, layer in enumerate(model.model.layers):
            if self.layers is None or i in self.layers:
                self._handles.append(layer.register_forward_hook(self._layer_hook(i)))
        self._handles.append(model.register_forward_hook(self._logits_hook))
        return self

    def _layer_hook(self, i):
        def hook(_mod, _inp, out):
            h, residual = out
            if isinstance(h, torch.Tensor) and isinstance(residual, torch.Tensor) and h.shape == residual.shape:
                self._cur[f"layer{i}.hidden"] = (h.float() + residual.float()).cpu()
        return hook

    def _logits_hook(self, _mod, _inp, out):
        from ..checkpoint.safetensors_io import save_file
        if isinstance(out, torch.Tensor):
            self._cur["logits"] = out.float().cpu()
        save_file(self._cur, os.path.join(self.out_dir, f"step{self.step}.safetensors"))
        self._cur = {}
        self.step += 1

    def detach(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []


def forced_tokens_from_env() -> Optional[List[List[int]]]:
    p = os.environ.get("TELB_FORCE_TOKENS_FILE")
    if not p:
        return None
    with open(p, "r", encoding="utf-8") as f:
        rows = json.load(f)
    return [[int(t) for t in r] for r in rows]
