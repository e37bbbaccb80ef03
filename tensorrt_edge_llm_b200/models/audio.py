"""Audio encoder (Whisper / Qwen2-Audio style) producing embedding rows for the language model.

Log-mel frames ``[n_mels, T]`` → two 3-tap convolutions (the second with stride 2) with GELU → fixed sinusoidal
positions → pre-LayerNorm transformer blocks with bidirectional attention → LayerNorm → optional average pooling by 2
and a linear projector into the LLM's hidden size.  The convolutions run as im2col + the tcgen05 GEMM, the blocks
are the vision encoder's (:class:`~.vit.VitBlock`: paged tile attention kernel with the causal mask off).

Parity: the audio towers of ``tensorrt_edgellm/models`` (Qwen2-Audio / Qwen3-Omni audio encoder, Whisper-derived ASR
encoders), built by ``cpp/builder/audioBuilder.cpp`` and fed by ``cpp/runtime/melSpectrogram.cpp`` in the reference.
Checkpoint names follow the Hugging Face Whisper encoder (``conv1``, ``conv2``, ``embed_positions``,
``layers.N.{self_attn.{q,k,v,out}_proj, self_attn_layer_norm, fc1, fc2, final_layer_norm}``, ``layer_norm``)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch
from torch import nn

from .. import ops
from ..ops.meta import build_step_meta
from .vit import VisionConfig, VitBlock, _LayerNorm, _Linear


@dataclass
class AudioConfig:
    n_mels: int = 128
    hidden_size: int = 1280
    num_hidden_layers: int = 32
    num_attention_heads: int = 20
    intermediate_size: int = 5120
    max_source_positions: int = 1500          # positions after the stride-2 convolution
    layer_norm_eps: float = 1e-5
    avg_pool: int = 2                          # 1 = none (plain Whisper encoder output)
    out_hidden_size: int = 0                   # 0 = no projector
    dtype: str = "bfloat16"

    @property
    def compute_dtype(self) -> torch.dtype:
        return getattr(torch, self.dtype)

    def block_config(self) -> VisionConfig:
        return VisionConfig(hidden_size=self.hidden_size, num_hidden_layers=self.num_hidden_layers,
                            num_attention_heads=self.num_attention_heads, intermediate_size=self.intermediate_size,
                            layer_norm_eps=self.layer_norm_eps, gelu_tanh=False, dtype=self.dtype)


def sinusoid_positions(length: int, channels: int) -> torch.Tensor:
    """Whisper's fixed table: ``[sin(t · w_i) ‖ cos(t · w_i)]`` with log-spaced timescales up to 10000."""
    inc = math.log(10000.0) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2, dtype=torch.float32))
    t = torch.arange(length, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([t.sin(), t.cos()], dim=1)


def _im2col_k3(x: torch.Tensor, stride: int) -> torch.Tensor:
    """``x [B, T, C]`` → ``[B, T_out, 3·C]`` windows of a 3-tap, padding-1 convolution (tap-major columns)."""
    b, t, c = x.shape
    xp = torch.nn.functional.pad(x, (0, 0, 1, 1))
    t_out = (t + 2 - 3) // stride + 1
    idx = torch.arange(t_out, device=x.device) * stride
    return torch.cat([xp[:, idx + k] for k in range(3)], dim=-1)


class AudioEncoder(nn.Module):
    """``forward(mel [B, n_mels, T])`` → ``[B · T_out, out]`` rows, ``T_out = T / 2 / avg_pool``."""

    def __init__(self, cfg: AudioConfig):
        super().__init__()
        bc = cfg.block_config()
        if bc.head_dim not in (64, 128):
            raise ValueError("the attention kernel takes head dimensions of 64 or 128")
        self.cfg = cfg
        dt, h = cfg.compute_dtype, cfg.hidden_size
        self.conv1, self.conv2 = _Linear(3 * cfg.n_mels, h, dt), _Linear(3 * h, h, dt)      # im2col form of the two convolutions
        self.register_buffer("embed_positions", sinusoid_positions(cfg.max_source_positions, h).to(dt))
        self.blocks = nn.ModuleList([VitBlock(bc) for _ in range(cfg.num_hidden_layers)])
        self.ln_post = _LayerNorm(h, cfg.layer_norm_eps, dt)
        self.proj = _Linear(h, cfg.out_hidden_size, dt) if cfg.out_hidden_size else None
        self._kv: Optional[torch.Tensor] = None

    @torch.no_grad()
    def random_init(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator().manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("weight") and p.dim() == 2:
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
        return self

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], prefix: str = "") -> None:
        """Fill from a Hugging Face Whisper-encoder style state dict (``prefix`` e.g. ``"audio_tower."``)."""
        def g(k):
            return sd[prefix + k]
        dt = self.cfg.compute_dtype
        # Conv1d weight [out, in, 3] → columns ordered tap-major to match the im2col layout
        self.conv1.weight.copy_(g("conv1.weight").permute(0, 2, 1).reshape(self.conv1.weight.shape).to(dt))
        self.conv1.bias.copy_(g("conv1.bias").to(dt))
        self.conv2.weight.copy_(g("conv2.weight").permute(0, 2, 1).reshape(self.conv2.weight.shape).to(dt))
        self.conv2.bias.copy_(g("conv2.bias").to(dt))
        if prefix + "embed_positions.weight" in sd:
            self.embed_positions.copy_(g("embed_positions.weight")[:self.embed_positions.shape[0]].to(dt))
        for i, blk in enumerate(self.blocks):
            p = f"layers.{i}."
            q, k, v = g(p + "self_attn.q_proj.weight"), g(p + "self_attn.k_proj.weight"), g(p + "self_attn.v_proj.weight")
            blk.qkv.weight.copy_(torch.cat([q, k, v], 0).to(dt))
            kb = sd.get(prefix + p + "self_attn.k_proj.bias", torch.zeros(k.shape[0]))      # Whisper's key projection has no bias
            blk.qkv.bias.copy_(torch.cat([g(p + "self_attn.q_proj.bias"), kb, g(p + "self_attn.v_proj.bias")], 0).to(dt))
            blk.proj.weight.copy_(g(p + "self_attn.out_proj.weight").to(dt)); blk.proj.bias.copy_(g(p + "self_attn.out_proj.bias").to(dt))
            blk.norm1.weight.copy_(g(p + "self_attn_layer_norm.weight").to(dt)); blk.norm1.bias.copy_(g(p + "self_attn_layer_norm.bias").to(dt))
            blk.norm2.weight.copy_(g(p + "final_layer_norm.weight").to(dt)); blk.norm2.bias.copy_(g(p + "final_layer_norm.bias").to(dt))
            blk.fc1.weight.copy_(g(p + "fc1.weight").to(dt)); blk.fc1.bias.copy_(g(p + "fc1.bias").to(dt))
            blk.fc2.weight.copy_(g(p + "fc2.weight").to(dt)); blk.fc2.bias.copy_(g(p + "fc2.bias").to(dt))
        self.ln_post.weight.copy_(g("layer_norm.weight").to(dt)); self.ln_post.bias.copy_(g("layer_norm.bias").to(dt))

    def _scratch_kv(self, pages: int, device) -> torch.Tensor:
        bc = self.blocks[0].cfg
        if self._kv is None or self._kv.shape[0] < pages or self._kv.device != device:
            self._kv = torch.zeros(pages, 2, bc.num_attention_heads, 64, bc.head_dim, dtype=self.cfg.compute_dtype, device=device)
        return self._kv

    @torch.no_grad()
    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        b, _, frames = mel.shape
        dev = mel.device
        x = mel.to(c.compute_dtype).transpose(1, 2).contiguous()                              # [B, T, mels]
        x = ops.gelu(self.conv1(_im2col_k3(x, 1).reshape(b * frames, -1)), False).view(b, frames, -1)
        t2 = (frames + 2 - 3) // 2 + 1
        if t2 > c.max_source_positions:
            raise ValueError(f"{frames} mel frames exceed the encoder's {2 * c.max_source_positions}")
        x = ops.gelu(self.conv2(_im2col_k3(x, 2).reshape(b * t2, -1)), False)
        x = x + self.embed_positions[:t2].repeat(b, 1)
        page = 64
        per = (t2 + page - 1) // page
        table = torch.arange(b * per, dtype=torch.int32).view(b, per)
        meta = build_step_meta([t2] * b, [0] * b, table, page, device=dev)
        kv = self._scratch_kv(b * per, dev)
        no_rope = torch.zeros(t2, 0, dtype=torch.float32, device=dev)
        for blk in self.blocks:
            x = blk(x, meta, kv, no_rope)
        x = self.ln_post(x)
        if c.avg_pool > 1:
            t3 = t2 // c.avg_pool
            x = x.view(b, t2, -1)[:, :t3 * c.avg_pool].reshape(b, t3, c.avg_pool, -1).float().mean(2).to(c.compute_dtype).reshape(b * t3, -1)
        return self.proj(x) if self.proj is not None else x


def audio_features(samples, sample_rate: int, n_mels: int = 128, chunk_seconds: int = 30) -> torch.Tensor:
    """Waveform → ``[1, n_mels, frames]`` log-mel input of the encoder (resampled to 16 kHz, padded to the chunk)."""
    import numpy as np
    from ..runtime import native as rt
    x = np.asarray(samples, dtype=np.float32)
    if sample_rate != 16000:
        x = rt.resample_linear(x, sample_rate, 16000)
    cfg = rt.MelConfig()
    cfg.n_mels = n_mels
    cfg.pad_to_samples = chunk_seconds * 16000
    return torch.from_numpy(np.ascontiguousarray(rt.log_mel_spectrogram(x, cfg)))[None]
