"""Flow-matching action expert of vision-language-action models (Alpamayo style).

After the vision-language model has read the scene and reasoned about it, a second, narrower transformer — the *expert* —
turns noise into a driving trajectory: ``n_diffusion_tokens`` waypoints of (acceleration, curvature).  The expert has
as many layers as the language model and the same key / value geometry, because layer ``i`` of the expert attends to
layer ``i`` of the language model's KV cache: its own rows are appended behind the cached context (without being
committed) and every waypoint row sees the whole context and every other waypoint (no causal mask).  One call is one
Euler step of the flow ``x ← x + (t1 - t0) · v(x, t0)``:

    waypoints + time → Fourier features → MLP encoder → LayerNorm → expert layers → RMSNorm → Linear(H → 2) = velocity

Here a step is one ragged engine step (``T`` rows per sequence, full tree mask) through the engine's GEMM, RoPE / KV-write
and attention kernels over the language model's own page pool; ``runtime/action.py`` drives the steps.

Parity: ``tensorrt_edgellm/models/alpamayo/modeling_alpamayo_action.py`` (``FourierEncoder`` :43, ``ActionInProjection``
:101, ``ActionAttention`` :145, ``AlpamayoAction.forward`` :336) and ``tensorrt_edgellm/config.py:380`` (``ActionConfig``)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..ops.meta import StepMeta
from ..parallel.comm import LocalComm
from .default import MLP, Attention, RMSNorm


@dataclass
class ActionConfig:
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 5_000_000.0
    attention_scaling: Optional[float] = None
    n_diffusion_tokens: int = 64
    num_traj_tokens: int = 1000
    traj_token_start: int = 0
    in_proj_hidden_size: int = 512
    in_proj_num_enc_layers: int = 2
    in_proj_max_freq: float = 100.0
    in_proj_num_fourier_feats: int = 20
    max_position_embeddings: int = 32768
    dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ActionConfig":
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in known})

    def model_config(self) -> ModelConfig:
        """The expert's transformer geometry in the terms the decoder modules are built from."""
        return ModelConfig(model_type="action_expert", vocab_size=8, hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
                           num_hidden_layers=self.num_hidden_layers, num_attention_heads=self.num_attention_heads,
                           num_key_value_heads=self.num_key_value_heads, head_dim=self.head_dim, rms_norm_eps=self.rms_norm_eps,
                           rope_theta=self.rope_theta, max_position_embeddings=self.max_position_embeddings, has_qk_norm=True, dtype=self.dtype)


class FourierEncoder(nn.Module):
    """``x → √2 · [sin(2π f x), cos(2π f x)]`` over ``dim / 2`` logarithmically spaced frequencies from 1 to ``max_freq``."""

    def __init__(self, dim: int, max_freq: float):
        super().__init__()
        self.out_dim = dim
        self.register_buffer("freqs", torch.logspace(0, math.log10(max_freq), steps=dim // 2)[None, :], persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        arg = x[..., None].float() * self.freqs.to(x.device) * (2 * math.pi)
        return torch.cat([torch.sin(arg), torch.cos(arg)], -1) * math.sqrt(2)


class _PlainRMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()


class ActionInProjection(nn.Module):
    """Waypoints ``[B, T, 2]`` and the flow time ``[B]`` → expert input rows ``[B · T, H]`` (fp32 math: a few thousand rows
    through a 512-wide MLP)."""

    def __init__(self, c: ActionConfig):
        super().__init__()
        nf = c.in_proj_num_fourier_feats
        self.sinus = nn.ModuleList([FourierEncoder(nf, c.in_proj_max_freq) for _ in range(2)])
        self.timestep_fourier_encoder = FourierEncoder(nf, c.in_proj_max_freq)
        layers: List[nn.Module] = [nn.Linear(3 * nf, c.in_proj_hidden_size), nn.SiLU()]
        for i in range(c.in_proj_num_enc_layers):
            last = i == c.in_proj_num_enc_layers - 1
            layers += [_PlainRMSNorm(c.in_proj_hidden_size, 1e-5), nn.Linear(c.in_proj_hidden_size, c.hidden_size if last else c.in_proj_hidden_size)]
            if not last:
                layers.append(nn.SiLU())
        self.encoder = nn.Sequential(*layers)
        self.norm = nn.LayerNorm(c.hidden_size)
        for p in self.parameters():
            p.requires_grad_(False)

    def forward(self, x: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        b, n, _ = x.shape
        feats = torch.cat([s(x[:, :, i]) for i, s in enumerate(self.sinus)], dim=-1)
        tf = self.timestep_fourier_encoder(t.reshape(b, 1)).expand(b, n, -1)
        h = torch.cat([feats, tf], dim=-1).reshape(b * n, -1)
        return self.norm(self.encoder(h))


class ActionExpertLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, scale: Optional[float]):
        super().__init__()
        p = f"layers.{idx}"
        self.self_attn = Attention(cfg, idx, f"{p}.self_attn")
        if scale:
            self.self_attn.scale = float(scale)
        self.mlp = MLP(cfg, f"{p}.mlp")
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)

    def forward(self, h, meta, kv_layer, cos_sin, comm):
        x = ops.rmsnorm(h, self.input_layernorm.weight, self.input_layernorm.eps)
        h = h + comm.all_reduce(self.self_attn(x, meta, kv_layer, cos_sin))
        x = ops.rmsnorm(h, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps)
        return h + comm.all_reduce(self.mlp(x))


class ActionExpert(nn.Module):
    """``velocity(x, t, meta, kv_pool)`` → ``[B, T, 2]``: the flow's velocity at waypoints ``x`` and time ``t``."""

    packed_modules = {"qkv_proj": ["q_proj", "k_proj", "v_proj"], "gate_up_proj": ["gate_proj", "up_proj"]}

    def __init__(self, action_cfg: ActionConfig, comm=None):
        super().__init__()
        self.action_cfg = action_cfg
        self.cfg = action_cfg.model_config()
        self.comm = comm or LocalComm()
        self.action_in_proj = ActionInProjection(action_cfg)
        self.layers = nn.ModuleList([ActionExpertLayer(self.cfg, i, action_cfg.attention_scaling) for i in range(self.cfg.num_hidden_layers)])
        self.norm = RMSNorm(self.cfg.hidden_size, self.cfg.rms_norm_eps, self.cfg.compute_dtype)
        self.action_out_proj = nn.Linear(self.cfg.hidden_size, 2, bias=True)
        for p in self.action_out_proj.parameters():
            p.requires_grad_(False)
        self._cos_sin: Optional[torch.Tensor] = None

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        """``expert.layers.N.mlp_gate_proj`` → ``layers.N.mlp.gate_proj`` and so on; the projections keep their names."""
        if key.startswith("expert."):
            key = key[len("expert."):]
            for flat in ("gate_proj", "up_proj", "down_proj"):
                key = key.replace(f".mlp_{flat}.", f".mlp.{flat}.")
        return key.replace("action_in_proj.encoder.trunk.", "action_in_proj.encoder.")

    @classmethod
    def from_pretrained(cls, expert_dir: str, device="cpu", comm=None) -> "ActionExpert":
        """Expert from a directory with ``config.json`` (the action hyper-parameters, at top level or under ``action_config``)
        and safetensors files in the reference's naming (``action_in_proj.*``, ``expert.layers.N.*``, ``action_out_proj.*``)."""
        import json
        import os
        from ..checkpoint.loader import load_weights
        with open(os.path.join(expert_dir, "config.json"), "r", encoding="utf-8") as f:
            d = json.load(f)
        model = cls(ActionConfig.from_dict(d.get("action_config", d)), comm)
        load_weights(model, expert_dir, strict=True)
        return model.to(device)

    def cos_sin(self, device) -> torch.Tensor:
        if self._cos_sin is None or self._cos_sin.device != torch.device(device):
            self._cos_sin = ops.rope_cos_sin(self.cfg.max_position_embeddings, self.cfg.rotary_dim, self.cfg.rope_theta, None, device=device)
        return self._cos_sin

    @torch.no_grad()
    def velocity(self, x: torch.Tensor, t: torch.Tensor, meta: StepMeta, kv_pool) -> torch.Tensor:
        b, n, _ = x.shape
        h = self.action_in_proj(x, t).to(self.cfg.compute_dtype)
        cs = self.cos_sin(h.device)
        for i, layer in enumerate(self.layers):
            h = layer(h, meta, kv_pool[i], cs, self.comm)
        h = ops.rmsnorm(h, self.norm.weight, self.norm.eps)
        return self.action_out_proj(h.float()).reshape(b, n, 2)

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.05):
        from ..checkpoint.loader import init_random_weights
        init_random_weights(self, seed, std)
        g = torch.Generator().manual_seed(seed + 1)
        for m in list(self.action_in_proj.modules()) + [self.action_out_proj]:
            if isinstance(m, nn.Linear):
                m.weight.copy_(torch.randn(m.weight.shape, generator=g) * std)
                m.bias.copy_(torch.randn(m.bias.shape, generator=g) * std)
        return self
