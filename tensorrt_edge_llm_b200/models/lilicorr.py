"""LiLiCorr draft: the DFlash 2 backbone with a candidate-lattice head.

Each of the ``S = block - 1`` proposal slots keeps its ``K`` most likely tokens.  The ``S · K`` candidates form a lattice; a
small bidirectional transformer over the lattice (additive attention bias from the slot distance, plus a same-slot term)
produces a state per candidate, from which three unit vectors are read — an *outgoing*, an *incoming* and, from the
sequence's anchor (the projected target hidden state of the last accepted token), an *anchor* vector.  The transition score
between candidate ``p`` of slot ``s - 1`` and candidate ``n`` of slot ``s`` is ``logit_scale · <out[s-1, p], in[s, n]>``; slot 0
is scored against the anchor.  The proposal is a walk over the lattice along those scores (``ops.lattice_chain_walk``).

A candidate's input node is the sum of: a projection of its token embedding (the target's table), a projection of the slot's
draft hidden state, an MLP of five per-candidate features (log-probability, probability, gap to the slot's best, rank
fraction, is-top-1; layer-normed), a slot embedding and a rank embedding.

The head works in fp32 on 16-bit weights.  The reference scales the backbone's sublayer outputs by 1/1024 (and the fusing
projection's input by 1/64) to stay inside fp16 range in its engine; those scalings cancel algebraically and are not
reproduced here, where the residual stream is not confined to fp16.

Parity: ``tensorrt_edgellm/models/lilicorr/modeling_lilicorr_head.py`` (bias :36-49, node features :262-283, factor heads
:296-339), ``tensorrt_edgellm/models/lilicorr/modeling_lilicorr_draft.py`` (anchor rows :33-52, head inputs :139-156),
``cpp/kernels/speculative/lilicorrChainWalk.h``; checkpoint tensors live under ``lilicorr.``."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from .default import RMSNorm
from .dflash import DFlashDraft
from .dflash2 import DFlash2Layer
from .linear import TPMode, make_linear

_FEATURES = 5
_FEATURE_EPS = 1e-5


def _lin(m: nn.Module, x: torch.Tensor) -> torch.Tensor:
    """fp32 product with a (16-bit) dense layer's weight and bias."""
    b = getattr(m, "bias", None)
    return F.linear(x.float(), m.weight.float(), None if b is None else b.float())


def _rms(m: RMSNorm, x: torch.Tensor) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + m.eps) * m.weight.float()


def _unit(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / v.pow(2).sum(-1, keepdim=True).sqrt().clamp_min(eps)


def lattice_attention_bias(relative_slot_bias: torch.Tensor, same_slot_bias: torch.Tensor, slots: int, topk: int, block: int) -> torch.Tensor:
    """``bias[h, q, k] = relative_slot_bias[h, slot(q) - slot(k) + block - 1] + same_slot_bias[h] · [slot(q) == slot(k)]`` with
    ``slot(i) = i // topk``; fp32 ``[heads, slots · topk, slots · topk]``."""
    slot = torch.arange(slots, device=relative_slot_bias.device).repeat_interleave(topk)
    dist = slot[:, None] - slot[None, :] + (block - 1)
    same = (slot[:, None] == slot[None, :]).float()
    return relative_slot_bias.float()[:, dist] + same_slot_bias.float()[:, None, None] * same


class _Mlp(nn.Module):
    def __init__(self, cfg, prefix, n_in, n_mid, n_out):
        super().__init__()
        self.up_proj = make_linear(cfg, f"{prefix}.up_proj", n_in, [n_mid], TPMode.REPLICATED, bias=True, quantizable=False)
        self.down_proj = make_linear(cfg, f"{prefix}.down_proj", n_mid, [n_out], TPMode.REPLICATED, bias=True, quantizable=False)

    def forward(self, x):
        return _lin(self.down_proj, F.silu(_lin(self.up_proj, x)))


class _FeatureNorm(nn.Module):
    def __init__(self, dt):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(_FEATURES, dtype=dt), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(_FEATURES, dtype=dt), requires_grad=False)


class _LatticeAttention(nn.Module):
    def __init__(self, cfg, prefix, hidden, heads):
        super().__init__()
        dt = cfg.compute_dtype
        self.heads, self.head_dim = heads, hidden // heads
        self.in_proj_weight = nn.Parameter(torch.zeros(3 * hidden, hidden, dtype=dt), requires_grad=False)
        self.in_proj_bias = nn.Parameter(torch.zeros(3 * hidden, dtype=dt), requires_grad=False)
        self.out_proj = make_linear(cfg, f"{prefix}.out_proj", hidden, [hidden], TPMode.REPLICATED, bias=True, quantizable=False)

    def forward(self, x, bias):
        b, n, hidden = x.shape
        qkv = F.linear(x, self.in_proj_weight.float(), self.in_proj_bias.float())
        q, k, v = (t.reshape(b, n, self.heads, self.head_dim).transpose(1, 2) for t in qkv.split(hidden, dim=-1))
        p = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(self.head_dim) + bias, dim=-1)
        return _lin(self.out_proj, (p @ v).transpose(1, 2).reshape(b, n, hidden))


class _LatticeLayer(nn.Module):
    def __init__(self, cfg, prefix, hidden, heads, mlp):
        super().__init__()
        dt = cfg.compute_dtype
        self.attn_norm = RMSNorm(hidden, cfg.rms_norm_eps, dt)
        self.attn = _LatticeAttention(cfg, f"{prefix}.attn", hidden, heads)
        self.mlp_norm = RMSNorm(hidden, cfg.rms_norm_eps, dt)
        self.mlp = _Mlp(cfg, f"{prefix}.mlp", hidden, mlp, hidden)

    def forward(self, x, bias):
        x = x + self.attn(_rms(self.attn_norm, x), bias)
        return x + self.mlp(_rms(self.mlp_norm, x))


class LiLiCorrHead(nn.Module):
    """``forward(token_embeddings [B, S, K, H], log_probs [B, S, K], slot_hidden [B, S, H], anchor [B, H], anchor_valid [B])``
    → transition scores ``[B, S, K(prev), K(next)]`` fp32, already multiplied by ``logit_scale``; slot 0 repeats the anchor
    scores for every ``prev``."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        hid, heads, dt = cfg.lilicorr_hidden_size, cfg.lilicorr_num_heads, cfg.compute_dtype
        if heads <= 0 or hid % heads:
            raise ValueError(f"LiLiCorr hidden size {hid} must be divisible by num_heads {heads}")
        self.block, self.slots, self.topk, self.hidden = cfg.dflash_block_size, cfg.dflash_block_size - 1, cfg.lilicorr_candidate_topk, hid
        self.vector_eps, self.logit_scale = cfg.lilicorr_vector_eps, cfg.lilicorr_logit_scale
        lin = lambda name, i, o: make_linear(cfg, f"lilicorr.{name}", i, [o], TPMode.REPLICATED, bias=True, quantizable=False)
        par = lambda *shape: nn.Parameter(torch.zeros(*shape, dtype=dt), requires_grad=False)
        self.token_proj = lin("token_proj", cfg.hidden_size, hid)
        self.pass_hidden_proj = lin("pass_hidden_proj", cfg.hidden_size, hid)
        self.feature_norm = _FeatureNorm(dt)
        self.feature_mlp = _Mlp(cfg, "lilicorr.feature_mlp", _FEATURES, hid, hid)
        self.slot_embedding = par(1, 1, self.slots, 1, hid)
        self.rank_embedding = par(1, 1, 1, self.topk, hid)
        self.relative_slot_bias = par(heads, 2 * self.block - 1)
        self.same_slot_bias = par(heads)
        self.context_proj = lin("context_proj", cfg.hidden_size, hid)
        self.layers = nn.ModuleList([_LatticeLayer(cfg, f"lilicorr.layers.{i}", hid, heads, int(hid * cfg.lilicorr_mlp_ratio))
                                     for i in range(cfg.lilicorr_num_layers)])
        self.output_norm = RMSNorm(hid, cfg.rms_norm_eps, dt)
        self.anchor_norm = RMSNorm(hid, cfg.rms_norm_eps, dt)
        self.factor_input_proj = lin("factor_input_proj", 3 * hid, hid)
        self.out_head = lin("out_head", hid, cfg.lilicorr_factor_dim)
        self.in_head = lin("in_head", hid, cfg.lilicorr_factor_dim)
        self.anchor_out_head = lin("anchor_out_head", hid, cfg.lilicorr_factor_dim)
        self._bias: Optional[torch.Tensor] = None

    def attention_bias(self) -> torch.Tensor:
        if self._bias is None or self._bias.device != self.relative_slot_bias.device:
            self._bias = lattice_attention_bias(self.relative_slot_bias, self.same_slot_bias, self.slots, self.topk, self.block)
        return self._bias

    def forward(self, token_embeddings, log_probs, slot_hidden, anchor, anchor_valid):
        b, k, hid = token_embeddings.shape[0], self.topk, self.hidden
        lp = log_probs.float()
        rank = torch.arange(k, dtype=torch.float32, device=lp.device)
        feats = torch.stack([lp, lp.exp(), lp - lp.amax(dim=-1, keepdim=True), (rank / float(max(k - 1, 1))).expand_as(lp),
                             (rank == 0).float().expand_as(lp)], dim=-1)
        feats = F.layer_norm(feats, (_FEATURES,), self.feature_norm.weight.float(), self.feature_norm.bias.float(), _FEATURE_EPS)
        nodes = (_lin(self.token_proj, token_embeddings) + _lin(self.pass_hidden_proj, slot_hidden)[:, :, None, :] + self.feature_mlp(feats)
                 + self.slot_embedding[0, 0].float() + self.rank_embedding[0, 0].float())
        x = nodes.reshape(b, self.slots * k, hid)
        bias = self.attention_bias()
        for layer in self.layers:
            x = layer(x, bias)
        states = _rms(self.output_norm, x).reshape(b, self.slots, k, hid)
        a = _rms(self.anchor_norm, _lin(self.context_proj, anchor) * anchor_valid.float()[:, None])
        # factor_input_proj reads concat(state, anchor, state · anchor): the anchor block of its weight is applied once per sequence
        w, bias_f = self.factor_input_proj.weight.float(), self.factor_input_proj.bias.float()
        ar = a[:, None, None, :]
        pre = F.linear(states, w[:, :hid], bias_f) + F.linear(ar, w[:, hid:2 * hid]) + F.linear(states * ar, w[:, 2 * hid:])
        factor = F.silu(pre)
        out_vec = _unit(_lin(self.out_head, factor), self.vector_eps)
        in_vec = _unit(_lin(self.in_head, factor), self.vector_eps)
        a_out = _unit(_lin(self.anchor_out_head, a), self.vector_eps)
        start = (in_vec[:, 0] @ a_out[:, :, None])[..., 0]                                    # [B, K]
        pair = out_vec[:, :-1] @ in_vec[:, 1:].transpose(-1, -2)                             # [B, S-1, K, K]
        return self.logit_scale * torch.cat([start[:, None, None, :].expand(b, 1, k, k), pair], dim=1)


@register_model("lilicorr", "lilicorr_draft")
class LiLiCorrDraft(DFlashDraft):
    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__(cfg, comm)
        if cfg.dflash_shift_label:
            raise ValueError("LiLiCorr drafts do not shift labels")
        self.layers = nn.ModuleList([DFlash2Layer(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.lilicorr = LiLiCorrHead(cfg)
        self._anchor: Dict[int, torch.Tensor] = {}             # per cache slot: projected context row of the last accepted token

    @torch.no_grad()
    def write_context(self, target_hidden: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor) -> None:
        h = self.project(target_hidden)
        cs = self.cos_sin(h.device)
        for i, layer in enumerate(self.layers):
            layer.write_context(h, meta, kv_pool[i], cs)
        last = h.index_select(0, (meta.q_start[1:] - 1).long().clamp_min(0))
        for j, (slot, q) in enumerate(zip(meta.slot_ids.tolist(), meta.q_len.tolist())):
            if q > 0:
                self._anchor[int(slot)] = last[j]

    def forget(self, slot: int) -> None:
        self._anchor.pop(int(slot), None)

    def lattice(self, hid: torch.Tensor, slots):
        """Candidates and transition scores of blocks whose proposal rows are ``hid [N, S, H]`` (normalised draft hidden states)."""
        n, s, h = hid.shape
        logits = self.head(hid.reshape(n * s, h)).reshape(n, s, -1)
        values, ids = logits.topk(self.lilicorr.topk, dim=-1)
        log_probs = values - torch.logsumexp(logits, dim=-1, keepdim=True)
        emb = F.embedding(ids, self.embed_tokens.weight)
        zero = torch.zeros(h, dtype=hid.dtype, device=hid.device)
        anchor = torch.stack([self._anchor.get(int(sl), zero) for sl in slots])
        valid = torch.tensor([int(sl) in self._anchor for sl in slots], device=hid.device)
        return ids, self.lilicorr(emb, log_probs, hid, anchor, valid)

    @torch.no_grad()
    def propose_tokens(self, embeds: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor, last_accepted: torch.Tensor, block: int,
                       temperatures: Optional[torch.Tensor] = None, uniforms: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.block_hidden(embeds, meta, kv_pool)
        n = x.shape[0] // block
        ids, scores = self.lattice(x.reshape(n, block, -1)[:, 1:, :], meta.slot_ids.tolist())
        tokens, _ = ops.lattice_chain_walk(ids, scores, temperatures, uniforms)
        return tokens
