"""DSpark draft: a DFlash-style block backbone whose proposals pass through a Markov head and a confidence head.

* **Markov head.**  The backbone scores every proposal position independently.  The Markov head adds a rank-``R`` bigram
  correction so that position ``i`` knows which token was chosen at ``i - 1``: ``corrected_i = logits_i + W2 · W1[prev]``
  (``W1 [V, R]`` embeds the previous token, ``W2 [V, R]`` reads it out).  The chain is walked left to right, greedy or sampled.
* **Confidence head.**  ``sigmoid(w · [hidden_i ; W1[prev_i]] + b)`` estimates the chance that position ``i`` survives
  verification.  The running product is the survival probability of a prefix; a schedule (``threshold`` or ``sps``) turns it
  into a proposal length per sequence, and the decoder verifies only that many draft tokens (a ragged verification step).

The backbone is the DFlash draft (labels shifted by default: row ``i`` of a block predicts position ``i + 1``).  On the GPU an
all-greedy chain runs as one fused correction + arg-max kernel per step (``csrc/kernels/speculative.cu``).

Parity: ``tensorrt_edgellm/models/dspark/modeling_dspark_draft.py`` (backbone), ``cpp/runtime/decoding/dsparkDecoder.cpp``
(sidecar tensors ``markov_w1`` / ``markov_w2`` / ``confidence_weight`` / ``confidence_bias`` :405-434, scheduler :150-170),
``cpp/kernels/speculative/dsparkKernels.cu`` (confidence :624-662, schedules :664-744, Markov logits :746-790)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from .dflash import DFlashDraft


@register_model("dspark", "dspark_draft")
class DSparkDraft(DFlashDraft):
    """``propose_tokens`` returns the Markov chain ``[N, block - 1]`` and leaves ``last_confidence [N, block - 1]`` and
    ``last_proposal_lengths [N]`` (None without a confidence head) for the decoder.  ``schedule`` is ``("threshold", t)`` or
    ``("sps", floor)``; ``min_proposal_len`` / ``max_proposal_len`` clamp the result."""

    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__(cfg, comm)
        if cfg.dspark_markov_rank <= 0:
            raise ValueError("DSpark requires a positive markov_rank")
        dt, r = cfg.compute_dtype, cfg.dspark_markov_rank
        mk = lambda *shape: nn.Parameter(torch.zeros(*shape, dtype=dt), requires_grad=False)
        self.markov_w1 = mk(cfg.vocab_size, r)
        self.markov_w2 = mk(cfg.vocab_size, r)
        self.with_confidence = bool(cfg.dspark_enable_confidence_head)
        self.confidence_with_markov = bool(cfg.dspark_confidence_head_with_markov)
        if self.with_confidence:
            self.confidence_weight = mk(cfg.hidden_size + (r if self.confidence_with_markov else 0))
            self.confidence_bias = mk(1)
        self.schedule = ("threshold", 0.0)                     # threshold 0: always the full block
        self.min_proposal_len, self.max_proposal_len = 1, 0
        self.last_confidence: Optional[torch.Tensor] = None
        self.last_proposal_lengths: Optional[torch.Tensor] = None

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        if "rotary_emb" in key or key in ("t2d", "d2t"):
            return None
        return DFlashDraft.checkpoint_key_remap(key)

    @torch.no_grad()
    def propose_tokens(self, embeds: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor, last_accepted: torch.Tensor, block: int,
                       temperatures: Optional[torch.Tensor] = None, uniforms: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.block_hidden(embeds, meta, kv_pool)
        n = x.shape[0] // block
        hid = x.reshape(n, block, -1)[:, 1:, :]
        logits = self.head(hid.reshape(n * (block - 1), -1)).reshape(n, block - 1, -1)
        tokens = ops.markov_chain_propose(logits, self.markov_w1, self.markov_w2, last_accepted, temperatures, uniforms)
        self.last_confidence = self.last_proposal_lengths = None
        if self.with_confidence:
            conf = ops.ref.markov_confidence(hid, self.markov_w1, self.confidence_weight, self.confidence_bias, last_accepted, tokens,
                                             self.confidence_with_markov)
            self.last_confidence = conf
            self.last_proposal_lengths = ops.ref.confidence_proposal_lengths(conf, self.schedule[0], float(self.schedule[1]),
                                                                             self.min_proposal_len, self.max_proposal_len)
        return tokens
