"""Reduced-vocabulary LM head: keep the tokens a deployment needs, map sampled ids back.

Parity: ``tensorrt_edgellm/vocab_reduction/`` and the sampler's reduced-vocab map
(``cpp/sampler/sampling.h``: logits over ``[reduced]`` columns, ``vocab_map[reduced] → full id``)."""
from __future__ import annotations

import json
import os
from typing import Iterable, List, Optional, Sequence

import torch

from ..checkpoint.safetensors_io import CheckpointReader, save_file


def build_vocab_map(vocab_size: int, token_counts: Optional[torch.Tensor] = None, keep: int = 0, always_keep: Sequence[int] = ()
                    ) -> torch.Tensor:
    """Sorted int32 ids of the kept tokens: ``always_keep`` (special tokens) plus the ``keep`` most frequent."""
    if keep <= 0 or keep >= vocab_size:
        return torch.arange(vocab_size, dtype=torch.int32)
    score = token_counts.double().clone() if token_counts is not None else torch.zeros(vocab_size, dtype=torch.float64)
    if score.numel() != vocab_size:
        raise ValueError("token_counts must have one entry per vocabulary id")
    score -= torch.arange(vocab_size, dtype=torch.float64) * 1e-9          # ties: lower id first
    forced = torch.tensor(sorted(set(int(t) for t in always_keep)), dtype=torch.long)
    score[forced] = float("inf")
    ids = torch.topk(score, max(keep, forced.numel())).indices
    return torch.sort(ids).values.to(torch.int32)


def count_tokens(token_id_rows: Iterable[Sequence[int]], vocab_size: int) -> torch.Tensor:
    counts = torch.zeros(vocab_size, dtype=torch.int64)
    for row in token_id_rows:
        counts += torch.bincount(torch.as_tensor(list(row), dtype=torch.long), minlength=vocab_size)[:vocab_size]
    return counts


def reduce_vocab(model_dir: str, out_dir: str, vocab_map: torch.Tensor) -> dict:
    """Write ``vocab_map.safetensors`` (``vocab_map [reduced] int32``, ``lm_head.weight [reduced, H]``) next to
    the checkpoint; the runtime multiplies by the reduced head and maps sampled columns through the map."""
    reader = CheckpointReader(model_dir)
    keys = set(reader.keys())
    head_key = "lm_head.weight" if "lm_head.weight" in keys else next(k for k in keys if k.endswith("embed_tokens.weight"))
    head = reader.get(head_key)
    os.makedirs(out_dir, exist_ok=True)
    save_file({"vocab_map": vocab_map.to(torch.int32), "lm_head.weight": head[vocab_map.long()].clone()},
              os.path.join(out_dir, "vocab_map.safetensors"))
    meta = {"full_vocab_size": int(head.shape[0]), "reduced_vocab_size": int(vocab_map.numel()), "source": head_key}
    with open(os.path.join(out_dir, "vocab_reduction.json"), "w", encoding="utf-8") as f:
        json.dump(meta, f, indent=1)
    return meta


def map_to_full(sampled: torch.Tensor, vocab_map: torch.Tensor) -> torch.Tensor:
    return vocab_map.to(sampled.device)[sampled.long()]
