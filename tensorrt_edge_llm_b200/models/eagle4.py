"""EAGLE-4 draft head: the EAGLE-3 single-layer draft with three optional additions.

* ``fc_norm``: every tapped target layer's hidden state gets an RMSNorm of its own before the fusing projection ``fc``.
* ``norm_output``: the feature handed to the next draft step is the final-norm output, not the raw layer output.
* a low-rank candidate head: instead of a dense ``lm_head`` pass over the vocabulary, two thin factors
  (``down_proj [r, H]``, ``up_proj [V, r]``) pick ``draft_candidate_count`` tokens, whose exact logits then come from
  their ``lm_head`` rows; the head's output is the sorted candidate ids with a log-softmax over the candidate set.

The tree decoder (``runtime/speculative.py``) reads a draft's proposals through ``pick``; the candidate form packs the
two outputs into one tensor ``[rows, 2, Kc]`` (log-probabilities, ids as exact fp32 integers) so the per-seat state it
keeps between rounds stays one tensor per seat.

Parity: ``tensorrt_edgellm/models/eagle4/modeling_eagle4_draft.py`` (checkpoint layout :24-37, ``_fuse_target_hidden``,
``_draft_head``), ``tensorrt_edgellm/models/candidate_head.py``, key remap ``tensorrt_edgellm/model.py:1219-1243``
(``efficient_lm_head_down_proj.*`` / ``efficient_lm_head.*`` factors, ``embed_tokens`` skipped).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from .default import RMSNorm
from .eagle3 import Eagle3Draft
from .linear import TPMode, make_linear


class LowRankCandidateHead(nn.Module):
    """``down_proj [r, H]`` and ``up_proj [V, r]``; ``forward(normed hidden, lm_head weight)`` → ``(ids, log-probabilities)``."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.num_candidates = cfg.draft_candidate_count
        self.down_proj = make_linear(cfg, "candidate_head.down_proj", cfg.hidden_size, [cfg.draft_candidate_rank], TPMode.REPLICATED,
                                     quantizable=False)
        self.up_proj = make_linear(cfg, "candidate_head.up_proj", cfg.draft_candidate_rank, [cfg.vocab_size], TPMode.REPLICATED,
                                   quantizable=False)

    def forward(self, nrm: torch.Tensor, lm_head_weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return ops.low_rank_candidate_head(nrm, self.down_proj.weight, self.up_proj.weight, lm_head_weight, self.num_candidates)


@register_model("eagle4", "eagle4_draft")
class Eagle4Draft(Eagle3Draft):
    """Same call as :class:`Eagle3Draft`.  With a candidate head the first output is ``[rows, 2, Kc]`` (see the module
    docstring) and the draft vocabulary is the target's."""

    def __init__(self, cfg: ModelConfig, comm=None):
        if cfg.draft_candidate_count > 0:
            if (cfg.draft_vocab_size or cfg.vocab_size) != cfg.vocab_size:
                raise ValueError("an EAGLE candidate head scores the full vocabulary: draft_vocab_size must equal vocab_size")
            if not cfg.eagle_norm_output:
                raise ValueError("an EAGLE candidate head requires norm_output")
        super().__init__(cfg, comm)
        ht = cfg.eagle3_target_hidden_size or cfg.hidden_size
        self.target_hidden = ht
        self.fc_norm = (nn.ModuleList([RMSNorm(ht, cfg.rms_norm_eps, cfg.compute_dtype) for _ in range(cfg.eagle3_num_target_layers)])
                        if cfg.eagle_fc_norm else None)
        self.candidate_head = LowRankCandidateHead(cfg) if cfg.draft_candidate_count > 0 else None
        self.softcap = getattr(cfg, "final_logit_softcapping", None) or None

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        if key.startswith("embed_tokens."):                       # the draft reads the target's embedding
            return None
        for src, dst in (("efficient_lm_head_down_proj.", "candidate_head.down_proj."), ("efficient_lm_head.", "candidate_head.up_proj.")):
            if key.startswith(src):
                return dst + key[len(src):]
        return Eagle3Draft.checkpoint_key_remap(key)

    def pick(self, lp: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.candidate_head is None:
            return super().pick(lp, k)
        kc = self.candidate_head.num_candidates
        if lp.shape[-1] == 2 * kc:                                  # a caller flattened the (log-probability, id) pair
            lp = lp.reshape(*lp.shape[:-1], 2, kc)
        k = min(k, kc)
        # already ordered by log-probability: the best k are the first k
        return lp[..., 0, :k], lp[..., 1, :k].long()

    def forward(self, embeds: torch.Tensor, feature: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor):
        if feature.shape[-1] != self.cfg.hidden_size:
            if self.fc_norm is not None:
                chunks = feature.split(self.target_hidden, dim=-1)
                feature = torch.cat([n(c) for n, c in zip(self.fc_norm, chunks)], dim=-1)
            feature = self.fc(feature)
        h = self.layers[0](feature, embeds, meta, kv_pool[0], self.cos_sin(embeds.device), self.comm)
        if self.cfg.eagle_norm_output:
            h = self.norm(h)                                       # the fed-back feature is the normed output, for every row
            nrm = h if meta.logits_idx.numel() == h.shape[0] else h.index_select(0, meta.logits_idx.long())
        else:
            rows = h if meta.logits_idx.numel() == h.shape[0] else h.index_select(0, meta.logits_idx.long())
            nrm = self.norm(rows)
        if self.candidate_head is not None:
            ids, clp = self.candidate_head(nrm, self.lm_head.weight)
            return torch.stack((clp, ids.float()), dim=-2), h
        logits = self.lm_head(nrm).float()
        if self.softcap:
            logits = torch.tanh(logits / self.softcap) * self.softcap
        return torch.log_softmax(logits, dim=-1), h
