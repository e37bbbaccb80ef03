"""EAGLE-3 draft head.

One decoder layer that predicts the next token from two streams: the embedding of the token at
position ``i + 1`` and a feature for position ``i`` — either the target model's hidden states of
three tapped layers projected by ``fc [H, 3·H_target]``, or the draft's own output of the parent
node while a draft tree is being grown.  The attention input is the concatenation of the two
normalised streams (``2H`` wide); the residual stream is the feature.  The LM head covers a reduced
draft vocabulary mapped to target ids through ``d2t``.

Parity: ``tensorrt_edgellm/models/eagle3/modeling_eagle3_draft.py`` — checkpoint layout (:24-37:
``fc``, ``midlayer.*`` → ``layers.0.*``, ``norm``, ``lm_head``, ``d2t`` offsets), layer body
(:317-367), model forward with log-softmax outputs (:604-660).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from ..parallel.comm import LocalComm
from .default import MLP, RMSNorm
from .linear import TPMode, make_linear


class Eagle3Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        tp = cfg.tp_size
        self.head_dim = cfg.head_dim
        self.num_q_heads = cfg.num_attention_heads // tp
        self.num_kv_heads = max(cfg.num_key_value_heads // tp, 1)
        self.scale = cfg.head_dim ** -0.5
        self.eps = cfg.rms_norm_eps
        self.qkv_proj = make_linear(cfg, f"{prefix}.qkv_proj", 2 * cfg.hidden_size, [cfg.q_size, cfg.kv_size, cfg.kv_size],
                                    TPMode.COL, sources=["q_proj", "k_proj", "v_proj"], bias=cfg.attention_bias)
        self.o_proj = make_linear(cfg, f"{prefix}.o_proj", cfg.q_size, [cfg.hidden_size], TPMode.ROW)

    def forward(self, x2h: torch.Tensor, meta: StepMeta, kv_layer: torch.Tensor, cos_sin: torch.Tensor) -> torch.Tensor:
        qkv = self.qkv_proj(x2h)
        q = ops.rope_kv_write(qkv, kv_layer, meta, cos_sin, self.num_q_heads, self.num_kv_heads, self.head_dim, None, None, self.eps)
        o = ops.paged_attention(q, kv_layer, meta, self.scale, None)
        return self.o_proj(o.reshape(o.shape[0], -1))


class Eagle3Layer(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        dt = cfg.compute_dtype
        self.norm_before_residual = cfg.eagle3_norm_before_residual
        self.self_attn = Eagle3Attention(cfg, f"{prefix}.self_attn")
        self.mlp = MLP(cfg, f"{prefix}.mlp")
        self.hidden_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dt)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dt)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dt)

    def forward(self, feature, embeds, meta, kv_layer, cos_sin, comm):
        nh = self.hidden_norm(feature)
        ne = self.input_layernorm(embeds)
        residual = nh if self.norm_before_residual else feature
        a = self.self_attn(torch.cat((ne, nh), dim=-1), meta, kv_layer, cos_sin)
        x, residual = comm.add_rmsnorm(a, residual, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps)
        m = self.mlp(x)
        if comm.world_size > 1:
            m = comm.all_reduce(m)
        return m + residual


@register_model("eagle3", "eagle3_draft")
class Eagle3Draft(nn.Module):
    """``forward(embeds, feature, meta, kv_pool)`` → ``(log-probabilities over the draft vocabulary
    for meta.logits_idx rows, hidden output of every row)``.  ``feature`` is ``[T, H]`` (draft
    hidden of the parent) or ``[T, 3·H_target]`` (tapped target hidden states, projected here)."""

    packed_modules = {"qkv_proj": ["q_proj", "k_proj", "v_proj"], "gate_up_proj": ["gate_proj", "up_proj"]}

    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__()
        self.cfg = cfg
        self.comm = comm or LocalComm()
        ht = cfg.eagle3_target_hidden_size or cfg.hidden_size
        self.fc = make_linear(cfg, "fc", cfg.eagle3_num_target_layers * ht, [cfg.hidden_size], TPMode.REPLICATED, quantizable=False)
        self.layers = nn.ModuleList([Eagle3Layer(cfg, "layers.0")])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)
        dv = cfg.draft_vocab_size or cfg.vocab_size
        self.lm_head = make_linear(cfg, "lm_head", cfg.hidden_size, [dv], TPMode.REPLICATED, quantizable=False)
        self.register_buffer("d2t", torch.arange(dv, dtype=torch.int32))        # draft id → target id
        self._cos_sin: Optional[torch.Tensor] = None

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        """``midlayer.*`` is the single decoder layer; ``t2d`` is not needed at run time."""
        if key.startswith("t2d"):
            return None
        if key.startswith("midlayer."):
            return "layers.0." + key[len("midlayer."):]
        return key

    def finalize_checkpoint(self):
        """Hugging Face EAGLE-3 repositories store ``d2t`` as offsets (target = draft + d2t[draft])."""
        d = self.d2t.long()
        if d.numel() and int(d[0]) == 0 and not torch.equal(d, torch.arange(d.numel(), device=d.device)):
            self.d2t.copy_((d + torch.arange(d.numel(), device=d.device)).to(torch.int32))

    def pick(self, lp: torch.Tensor, k: int):
        """The ``k`` best proposals of each row of the head's output: ``(log-probabilities [..., k], target token ids [..., k])``."""
        sc, idx = lp.topk(min(k, lp.shape[-1]), dim=-1)
        return sc, self.d2t.long()[idx]

    def cos_sin(self, device) -> torch.Tensor:
        if self._cos_sin is None or self._cos_sin.device != torch.device(device):
            self._cos_sin = ops.rope_cos_sin(self.cfg.max_position_embeddings, self.cfg.rotary_dim, self.cfg.rope_theta,
                                                 self.cfg.rope_scaling, device=device)
        return self._cos_sin

    def forward(self, embeds: torch.Tensor, feature: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor):
        if feature.shape[-1] != self.cfg.hidden_size:
            feature = self.fc(feature)
        h = self.layers[0](feature, embeds, meta, kv_pool[0], self.cos_sin(embeds.device), self.comm)
        rows = h if meta.logits_idx.numel() == h.shape[0] else h.index_select(0, meta.logits_idx.long())
        logits = self.lm_head(self.norm(rows)).float()
        return torch.log_softmax(logits, dim=-1), h
