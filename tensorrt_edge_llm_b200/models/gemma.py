"""Gemma 3 style text decoder.

Differences from the Llama-style stack (``models/default.py``): four norms per layer (the attention and MLP outputs
are normalised *before* they join the residual stream), GeGLU MLP (tanh GELU), RMSNorm weights stored as ``w - 1``,
embeddings scaled by ``sqrt(hidden)``, attention scale ``query_pre_attn_scalar ** -0.5``, q / k norms, and a layer
pattern that alternates sliding-window layers (own RoPE base) with full-attention layers.  The stored-minus-one norm
weights and the embedding scale are folded into the tensors when a checkpoint is loaded, so the forward pass uses the
ordinary kernels.

Parity: ``tensorrt_edgellm/models/gemma4/`` (text stack) and the Hugging Face ``Gemma3ForCausalLM`` the tests use as
the numerical oracle.  Head dimensions other than 64 / 128 (Gemma's released checkpoints use 256) run on the PyTorch
reference ops only: the tcgen05 attention kernels are built for 64 and 128."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from .default import MLP, Attention, CausalLM, RMSNorm


class GemmaAttention(Attention):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__(cfg, layer_idx, prefix)
        if cfg.query_pre_attn_scalar:
            self.scale = cfg.query_pre_attn_scalar ** -0.5
        win = cfg.layer_windows[layer_idx] if cfg.layer_windows else (cfg.sliding_window or 0)
        self.sliding_window = win or None
        self.local_rope = bool(win) and cfg.rope_local_theta > 0


class GemmaMLP(MLP):
    def __init__(self, cfg: ModelConfig, prefix: str):
        act, cfg.hidden_act = cfg.hidden_act, "silu"              # build the fused gate‖up projection of the gated form
        try:
            super().__init__(cfg, prefix)
        finally:
            cfg.hidden_act = act
        self.tanh = "tanh" in act

    def forward(self, x):
        return self.down_proj(ops.geglu(self.gate_up_proj(x), self.tanh))


class GemmaLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int):
        super().__init__()
        p = f"model.layers.{layer_idx}"
        self.self_attn = GemmaAttention(cfg, layer_idx, f"{p}.self_attn")
        self.mlp = GemmaMLP(cfg, f"{p}.mlp")
        mk = lambda: RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)
        self.input_layernorm, self.post_attention_layernorm = mk(), mk()
        self.pre_feedforward_layernorm, self.post_feedforward_layernorm = mk(), mk()

    def forward(self, h, residual, meta, kv_layer, cos_sin, comm):
        if residual is None:
            residual = h
            x = ops.rmsnorm(h, self.input_layernorm.weight, self.input_layernorm.eps)
        else:
            x, residual = ops.add_rmsnorm(h, residual, self.input_layernorm.weight, self.input_layernorm.eps)
        a = comm.all_reduce(self.self_attn(x, meta, kv_layer, cos_sin[1] if self.self_attn.local_rope else cos_sin[0]))
        a = ops.rmsnorm(a, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps)
        x, residual = ops.add_rmsnorm(a, residual, self.pre_feedforward_layernorm.weight, self.pre_feedforward_layernorm.eps)
        m = comm.all_reduce(self.mlp(x))
        return ops.rmsnorm(m, self.post_feedforward_layernorm.weight, self.post_feedforward_layernorm.eps), residual


class GemmaTransformer(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=cfg.compute_dtype)
        self.embed_tokens.weight.requires_grad_(False)
        self.layers = nn.ModuleList([GemmaLayer(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)
        # multiplier applied after the lookup; a loaded checkpoint folds it into the table instead (see finalize_checkpoint)
        self.embed_scale = float(cfg.hidden_size) ** 0.5

    def forward(self, ids, meta, kv_cache, cos_sin, comm, inputs_embeds=None, capture_layers=()):
        if inputs_embeds is None:
            h = ops.embedding(ids, self.embed_tokens.weight)
            if self.embed_scale != 1.0:
                h = (h * torch.tensor(self.embed_scale, dtype=h.dtype)).to(h.dtype)
        else:
            h = inputs_embeds
        residual = None
        taps = []
        for i, layer in enumerate(self.layers):
            donor = layer.self_attn.kv_donor                 # KV-shared layers (num_kv_shared_layers) read an earlier layer's cache
            h, residual = layer(h, residual, meta, kv_cache[donor if donor >= 0 else i], cos_sin, comm)
            if i in capture_layers:
                taps.append((h.float() + residual.float()).to(h.dtype))
        x, _ = ops.add_rmsnorm(h, residual, self.norm.weight, self.norm.eps)
        return (x, taps) if capture_layers else x


@register_model("gemma3_text", "gemma3", "gemma2", "gemma")
class GemmaCausalLM(CausalLM):
    transformer_cls = GemmaTransformer

    def cos_sin(self, device):
        if self._cos_sin is None or self._cos_sin[0].device != torch.device(device):
            c = self.cfg
            full = ops.rope_cos_sin(c.max_position_embeddings, c.rotary_dim, c.rope_theta, c.rope_scaling, device=device)
            local = full if c.rope_local_theta <= 0 else ops.rope_cos_sin(c.max_position_embeddings, c.rotary_dim, c.rope_local_theta,
                                                                                c.rope_local_scaling, device=device)
            self._cos_sin = (full, local)
        return self._cos_sin

    def logits_from_hidden(self, x: torch.Tensor, meta: StepMeta) -> torch.Tensor:
        logits = super().logits_from_hidden(x, meta)
        cap = self.cfg.final_logit_softcapping
        if cap:
            logits = (torch.tanh(logits.float() / cap) * cap).to(logits.dtype)
        return logits

    @torch.no_grad()
    def finalize_checkpoint(self):
        """Checkpoint conventions → kernel conventions: norm weights are stored minus one, and the embedding rows are
        scaled by sqrt(hidden) at lookup (the LM head, tied to the same table, is copied before the scaling)."""
        for m in self.modules():
            if isinstance(m, RMSNorm):
                m.weight.add_(1.0)
        t = self.model
        t.embed_tokens.weight.mul_(torch.tensor(t.embed_scale, dtype=t.embed_tokens.weight.dtype))
        t.embed_scale = 1.0

    def artifacts_loaded(self):
        """Prepared weights already carry the folded norm offsets and the scaled embedding table."""
        self.model.embed_scale = 1.0
