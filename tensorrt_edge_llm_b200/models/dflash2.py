"""DFlash 2 block draft: the DFlash backbone with a dynamic convolution around every sublayer and a chain selector.

* Every attention and MLP sublayer is wrapped by a *dynamic grouped depthwise convolution* along the proposal block.  A
  projection of the normalised sublayer input yields, per token, ``2 · K · (H / group)`` filter offsets: the first half
  filters the sublayer's input (``prepare``), the second half filters its output before the residual add (``finish``).
  A filter tap is ``base[side, k, c] + offset[t, k, c // group]``; taps reach back ``K - 1`` rows and never leave the block.
* The head does not take each slot's arg-max independently.  Each slot keeps its ``top_k`` candidates with their (scaled,
  soft-capped) logits, and a *selector* walks the slots in order: a candidate's score is its logit plus a bilinear term
  ``<P[prev] ⊙ z_slot, Q[candidate]>`` between the token chosen for the previous slot (the last accepted token for the first
  slot), the slot's projected hidden state ``z`` and two ``[V, rank]`` codebooks.

Both run as one kernel each on the GPU (``csrc/kernels/speculative.cu``); everything else is the DFlash draft.

Parity: ``tensorrt_edgellm/models/dflash2/modeling_dflash2_draft.py`` (``DFlash2GroupedConv`` :36-90, layer :93-160, selector
parameters :163-180, head :270-300), ``cpp/kernels/speculative/dflash2GroupedDynamicConv.cu``,
``cpp/kernels/speculative/dflash2CandidateSelector.cu`` (chain walk)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from .dflash import DFlashDraft, DFlashLayer
from .linear import TPMode, make_linear


class GroupedDynamicConv(nn.Module):
    """``kernel_projection [2·K·G, H]`` (G = H / group size) and ``base_kernel [2, K, H]`` of one wrapped sublayer."""

    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        self.taps, self.group = cfg.dflash2_conv_kernel_size, cfg.dflash2_conv_group_size
        if cfg.hidden_size % self.group:
            raise ValueError("DFlash2 conv group_size must divide hidden_size")
        self.groups = cfg.hidden_size // self.group
        self.block = cfg.dflash_block_size
        self.kernel_projection = make_linear(cfg, f"{prefix}.kernel_projection", cfg.hidden_size, [2 * self.taps * self.groups],
                                             TPMode.REPLICATED, quantizable=False)
        self.base_kernel = nn.Parameter(torch.zeros(2, self.taps, cfg.hidden_size, dtype=cfg.compute_dtype), requires_grad=False)

    def prepare(self, x: torch.Tensor):
        """Filtered sublayer input and the offsets kept for ``finish``."""
        coef = self.kernel_projection(x)
        side = self.taps * self.groups
        pre = coef[:, :side].reshape(-1, self.taps, self.groups)
        post = coef[:, side:].reshape(-1, self.taps, self.groups)
        return ops.dflash2_grouped_dynamic_conv(x, pre, self.base_kernel[0], None, self.block, self.group), post

    def finish(self, y: torch.Tensor, post: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        return ops.dflash2_grouped_dynamic_conv(y, post, self.base_kernel[1], residual, self.block, self.group)


class DFlash2Layer(DFlashLayer):
    def __init__(self, cfg: ModelConfig, idx: int):
        super().__init__(cfg, idx)
        self.attention_conv = GroupedDynamicConv(cfg, f"layers.{idx}.attention_conv")
        self.mlp_conv = GroupedDynamicConv(cfg, f"layers.{idx}.mlp_conv")

    def forward(self, h, meta, kv_layer, cos_sin, comm):
        x = ops.rmsnorm(h, self.input_layernorm.weight, self.input_layernorm.eps)
        x, post = self.attention_conv.prepare(x)
        h = self.attention_conv.finish(comm.all_reduce(self.self_attn(x, meta, kv_layer, cos_sin)), post, h)
        x = ops.rmsnorm(h, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps)
        x, post = self.mlp_conv.prepare(x)
        return self.mlp_conv.finish(comm.all_reduce(self.mlp(x)), post, h)


@register_model("dflash2", "dflash2_draft")
class DFlash2Draft(DFlashDraft):
    """``propose_tokens`` returns the selector's chain ``[N, block - 1]``; the context write and the block pass are DFlash's."""

    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__(cfg, comm)
        if cfg.dflash_shift_label:
            raise ValueError("DFlash 2 drafts do not shift labels")
        self.layers = nn.ModuleList([DFlash2Layer(cfg, i) for i in range(cfg.num_hidden_layers)])
        r = cfg.dflash2_selector_rank
        self.hidden_projection = make_linear(cfg, "candidate_selector.hidden_projection", cfg.hidden_size, [r], TPMode.REPLICATED,
                                             quantizable=False)
        mk = lambda *shape: nn.Parameter(torch.zeros(*shape, dtype=cfg.compute_dtype), requires_grad=False)
        self.predecessor_codebook = mk(cfg.vocab_size, r)     # checkpoint: candidate_selector.predecessor_codebook
        self.successor_codebook = mk(cfg.vocab_size, r)       # candidate_selector.successor_codebook

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        key = DFlashDraft.checkpoint_key_remap(key)
        return {"candidate_selector.hidden_projection.weight": "hidden_projection.weight",
                "candidate_selector.predecessor_codebook": "predecessor_codebook",
                "candidate_selector.successor_codebook": "successor_codebook"}.get(key, key)

    def candidates(self, hid: torch.Tensor):
        """Per-slot support of the selector: ``(ids [N, S, K] int64, transformed logits [N, S, K] fp32, projected [N, S, R])``.
        The output multiplier and the soft cap are monotonic, so they are applied after the top-k."""
        n, s, _ = hid.shape
        flat = hid.reshape(n * s, -1)
        logits = self.lm_head(flat).float()
        unary, ids = logits.topk(min(self.cfg.dflash2_selector_top_k, logits.shape[-1]), dim=-1)
        if self.cfg.dflash2_output_multiplier != 1.0:
            unary = unary * self.cfg.dflash2_output_multiplier
        cap = self.cfg.final_logit_softcapping
        if cap:
            unary = torch.tanh(unary / cap) * cap
        z = self.hidden_projection(flat)
        return ids.reshape(n, s, -1), unary.reshape(n, s, -1), z.reshape(n, s, -1)

    @torch.no_grad()
    def propose_tokens(self, embeds: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor, last_accepted: torch.Tensor, block: int,
                       temperatures: Optional[torch.Tensor] = None, uniforms: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.block_hidden(embeds, meta, kv_pool)
        n = x.shape[0] // block
        ids, unary, z = self.candidates(x.reshape(n, block, -1)[:, 1:, :])
        tokens, _ = ops.dflash2_selector_walk(ids, unary, z, last_accepted, self.predecessor_codebook, self.successor_codebook,
                                              temperatures, uniforms)
        return tokens
