"""Multi-token-prediction (MTP) draft head.

``h = fc([norm_e(embed(token_{i+1})) ‖ norm_h(feature_i)])`` → one ordinary decoder layer → ``norm`` → LM head over
the full vocabulary (usually the target's own head).  The feature is the target's last hidden state for accepted
positions and the head's own output while a draft chain / tree grows, so the head plugs into the same
speculative decoder as the EAGLE-3 draft (``runtime/speculative.py``) with a single tapped layer.

Parity: ``tensorrt_edgellm/models/mtp/modeling_qwen3_mtp.py:15-60`` (tensor layout ``mtp.pre_fc_norm_embedding``,
``mtp.pre_fc_norm_hidden``, ``mtp.fc [H, 2H]``, ``mtp.layers.0``, ``mtp.norm``, shared ``lm_head``) and
``cpp/runtime/decoding/mtpDecoder.cpp`` (draft prefill → proposal → verify → accept-token)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from ..parallel.comm import LocalComm
from .default import DecoderLayer, RMSNorm
from .linear import TPMode, make_linear


@register_model("mtp", "qwen3_mtp")
class MtpDraft(nn.Module):
    """``forward(embeds, feature, meta, kv_pool)`` → (log-probabilities for ``meta.logits_idx`` rows, hidden of every row)."""

    packed_modules = {"qkv_proj": ["q_proj", "k_proj", "v_proj"], "gate_up_proj": ["gate_proj", "up_proj"]}

    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__()
        if cfg.num_hidden_layers != 1:
            raise ValueError("the MTP draft head has exactly one decoder layer")
        self.cfg = cfg
        self.comm = comm or LocalComm()
        h, dt = cfg.hidden_size, cfg.compute_dtype
        self.pre_fc_norm_embedding = RMSNorm(h, cfg.rms_norm_eps, dt)
        self.pre_fc_norm_hidden = RMSNorm(h, cfg.rms_norm_eps, dt)
        self.fc = make_linear(cfg, "fc", 2 * h, [h], TPMode.REPLICATED, quantizable=False)
        self.layers = nn.ModuleList([DecoderLayer(cfg, 0)])
        self.norm = RMSNorm(h, cfg.rms_norm_eps, dt)
        self.lm_head = make_linear(cfg, "lm_head", h, [cfg.vocab_size], TPMode.REPLICATED, quantizable=False)
        self.register_buffer("d2t", torch.arange(cfg.vocab_size, dtype=torch.int32))      # identity: full vocabulary
        self._cos_sin: Optional[torch.Tensor] = None

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        """Checkpoints prefix the head's tensors with ``mtp.``; decoder-layer names follow ``model.layers.0``."""
        if key.startswith("mtp."):
            key = key[len("mtp."):]
        if key.startswith("layers.0."):
            return "layers.0." + key[len("layers.0."):]
        return key

    def share_lm_head(self, target) -> None:
        """Use the target model's LM head (the usual arrangement: checkpoints do not duplicate it)."""
        self.lm_head = target.lm_head

    def cos_sin(self, device) -> torch.Tensor:
        if self._cos_sin is None or self._cos_sin.device != torch.device(device):
            self._cos_sin = ops.rope_cos_sin(self.cfg.max_position_embeddings, self.cfg.rotary_dim, self.cfg.rope_theta,
                                                 self.cfg.rope_scaling, device=device)
        return self._cos_sin

    def forward(self, embeds: torch.Tensor, feature: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor):
        x = self.fc(torch.cat((self.pre_fc_norm_embedding(embeds), self.pre_fc_norm_hidden(feature)), dim=-1))
        h, residual = self.layers[0](x, None, meta, kv_pool[0], self.cos_sin(embeds.device), self.comm)
        if self.comm.world_size > 1:
            h = self.comm.all_reduce(h)
        out = h + residual                                    # the layer returns (mlp output, residual stream)
        rows = out if meta.logits_idx.numel() == out.shape[0] else out.index_select(0, meta.logits_idx.long())
        logits = self.lm_head(self.norm(rows)).float()
        return torch.log_softmax(logits, dim=-1), out
