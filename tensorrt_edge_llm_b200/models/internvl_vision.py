"""InternVL vision tower (InternViT) with its pixel-shuffle projector.

A fixed-resolution ViT: patch embedding (the checkpoint's Conv2d has kernel = stride, so it is one GEMM over flat
patches), a class token that takes part in attention, learned position embeddings, pre-norm blocks whose attention and
MLP outputs are scaled per channel (``lambda_1`` / ``lambda_2``, "layer scale") before they join the residual stream,
optional RMS q / k normalisation over the whole embedding.  The language model receives ``(grid / 2)²`` rows per image
tile: the class token is dropped, 2 × 2 neighbouring patches are folded into the channel dimension (pixel shuffle) and a
LayerNorm → Linear → GELU → Linear projector maps them to the decoder's hidden size.

Attention runs the paged tile kernel with the causal mask off, each image tile being one sequence of ``1 + grid²`` rows
(``ops.paged_attention(..., causal=False)``), like ``models/vit.py``.

Parity: ``tensorrt_edgellm/models/internvl3`` / ``internvl3_5`` visual towers and ``cpp/multimodal/internViTRunner.cpp``
(tiles → embedding rows); the numerical oracle in the tests is Hugging Face ``InternVLModel.get_image_features``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
from torch import nn

from .. import ops
from ..ops.meta import build_step_meta


@dataclass
class InternVisionConfig:
    hidden_size: int = 1024
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    intermediate_size: int = 4096
    image_size: int = 448
    patch_size: int = 14
    num_channels: int = 3
    attention_bias: bool = False
    use_qk_norm: bool = False
    rms_norm: bool = False                   # norm_type "rms_norm" (the 6B tower) instead of LayerNorm
    layer_norm_eps: float = 1e-6
    final_layernorm: bool = False            # checkpoints with use_mean_pooling (the default) have none
    downsample_ratio: float = 0.5
    out_hidden_size: int = 4096              # the language model's hidden size
    dtype: str = "bfloat16"

    @classmethod
    def from_hf(cls, hf: Dict) -> "InternVisionConfig":
        """From a whole ``config.json`` (``vision_config``, ``text_config``, ``downsample_ratio``)."""
        v = hf["vision_config"]
        first = lambda x: int(x[0] if isinstance(x, (list, tuple)) else x)
        text = hf.get("text_config") or hf.get("llm_config") or {}
        return cls(hidden_size=int(v["hidden_size"]), num_hidden_layers=int(v["num_hidden_layers"]), num_attention_heads=int(v["num_attention_heads"]),
                   intermediate_size=int(v["intermediate_size"]), image_size=first(v.get("image_size", 448)), patch_size=first(v.get("patch_size", 14)),
                   num_channels=int(v.get("num_channels", 3)), attention_bias=bool(v.get("attention_bias", v.get("qkv_bias", False))),
                   use_qk_norm=bool(v.get("use_qk_norm", v.get("qk_normalization", False))), rms_norm=str(v.get("norm_type", "layer_norm")) == "rms_norm",
                   layer_norm_eps=float(v.get("layer_norm_eps", 1e-6)), final_layernorm=not bool(v.get("use_mean_pooling", True)),
                   downsample_ratio=float(hf.get("downsample_ratio", 0.5)), out_hidden_size=int(text.get("hidden_size", 4096)))

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def grid(self) -> int:
        return self.image_size // self.patch_size

    @property
    def compute_dtype(self) -> torch.dtype:
        return {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[self.dtype]


class _Lin(nn.Module):
    def __init__(self, i, o, dtype, bias=True):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(o, i, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype), requires_grad=False) if bias else None

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class _Norm(nn.Module):
    def __init__(self, dim, eps, dtype, rms):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.bias = None if rms else nn.Parameter(torch.zeros(dim, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps) if self.bias is None else ops.layernorm(x, self.weight, self.bias, self.eps)


class InternVisionBlock(nn.Module):
    def __init__(self, c: InternVisionConfig):
        super().__init__()
        dt, h = c.compute_dtype, c.hidden_size
        self.cfg = c
        self.norm1, self.norm2 = _Norm(h, c.layer_norm_eps, dt, c.rms_norm), _Norm(h, c.layer_norm_eps, dt, c.rms_norm)
        self.qkv = _Lin(h, 3 * h, dt, bias=True)               # checkpoints without attention bias keep it at zero
        self.proj = _Lin(h, h, dt)
        self.q_norm = _Norm(h, 1e-6, dt, True) if c.use_qk_norm else None
        self.k_norm = _Norm(h, 1e-6, dt, True) if c.use_qk_norm else None
        self.fc1, self.fc2 = _Lin(h, c.intermediate_size, dt), _Lin(c.intermediate_size, h, dt)
        self.lambda_1 = nn.Parameter(torch.ones(h, dtype=dt), requires_grad=False)
        self.lambda_2 = nn.Parameter(torch.ones(h, dtype=dt), requires_grad=False)

    def forward(self, x, meta, kv, no_rope):
        c = self.cfg
        qkv = self.qkv(self.norm1(x))
        if self.q_norm is not None:                              # RMS norm over the whole embedding, before the head split
            h = c.hidden_size
            qkv = torch.cat([self.q_norm(qkv[:, :h].contiguous()), self.k_norm(qkv[:, h:2 * h].contiguous()), qkv[:, 2 * h:]], dim=-1)
        q = ops.rope_kv_write(qkv, kv, meta, no_rope, c.num_attention_heads, c.num_attention_heads, c.head_dim)
        a = ops.paged_attention(q, kv, meta, c.head_dim ** -0.5, causal=False)
        x = x + self.lambda_1 * self.proj(a.reshape(a.shape[0], -1))
        return x + self.lambda_2 * self.fc2(ops.gelu(self.fc1(self.norm2(x))))


def tile_grid(width: int, height: int, tile: int, min_tiles: int = 1, max_tiles: int = 12):
    """Columns × rows of tiles for an image (the InternVL "dynamic resolution" rule): among all grids with
    ``min_tiles ≤ columns · rows ≤ max_tiles`` take the one whose aspect ratio is closest to the image's; on a tie the
    larger grid wins when the image has more than half of its pixels."""
    ratios = sorted({(i, j) for n in range(min_tiles, max_tiles + 1) for i in range(1, n + 1) for j in range(1, n + 1)
                     if min_tiles <= i * j <= max_tiles}, key=lambda r: r[0] * r[1])
    aspect = width / height
    best, best_diff = (1, 1), float("inf")
    for i, j in ratios:
        diff = abs(aspect - i / j)
        if diff < best_diff:
            best, best_diff = (i, j), diff
        elif diff == best_diff and width * height > 0.5 * tile * tile * i * j:
            best = (i, j)
    return best


class InternVisionEncoder(nn.Module):
    """``forward(pixels [N, C, S, S])`` (normalised tiles of the configured size) → ``[N · (grid · ratio)², out_hidden]``."""

    PAGE = 64
    image_mean = (0.485, 0.456, 0.406)
    image_std = (0.229, 0.224, 0.225)

    def __init__(self, cfg: InternVisionConfig):
        super().__init__()
        self.cfg = cfg
        dt, h = cfg.compute_dtype, cfg.hidden_size
        # the tensor-core GEMM wants a reduction length that is a multiple of 8 (16-byte rows): 3 · 14 · 14 = 588 is not, so
        # the patch matrix and the weight get zero columns up to the next multiple
        self.patch_dim = cfg.num_channels * cfg.patch_size ** 2
        self.patch_pad = (-self.patch_dim) % 8
        self.patch_embed = _Lin(self.patch_dim + self.patch_pad, h, dt)
        self.cls_token = nn.Parameter(torch.zeros(h, dtype=dt), requires_grad=False)
        self.pos_embed = nn.Parameter(torch.zeros(1 + cfg.grid ** 2, h, dtype=dt), requires_grad=False)
        self.blocks = nn.ModuleList([InternVisionBlock(cfg) for _ in range(cfg.num_hidden_layers)])
        self.norm = _Norm(h, cfg.layer_norm_eps, dt, False) if cfg.final_layernorm else None
        fold = int(round(1 / cfg.downsample_ratio)) ** 2
        self.proj_norm = _Norm(h * fold, 1e-5, dt, False)
        self.proj_fc1, self.proj_fc2 = _Lin(h * fold, cfg.out_hidden_size, dt), _Lin(cfg.out_hidden_size, cfg.out_hidden_size, dt)
        self._kv: Optional[torch.Tensor] = None

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], tower: str = "vision_tower.", projector: str = "multi_modal_projector.") -> List[str]:
        """Fill from Hugging Face ``InternVLModel`` tensors; returns the names under the two prefixes that were not used."""
        c = self.cfg
        used = set()

        def take(name):
            used.add(name)
            return sd[name]

        def put(param, value):
            if tuple(param.shape) != tuple(value.shape):
                raise ValueError(f"shape {tuple(value.shape)} does not fit {tuple(param.shape)}")
            param.copy_(value.to(param.dtype))
        e = tower + "embeddings."
        put(self.patch_embed.weight, torch.nn.functional.pad(take(e + "patch_embeddings.projection.weight").reshape(c.hidden_size, -1),
                                                             (0, self.patch_pad)))
        put(self.patch_embed.bias, take(e + "patch_embeddings.projection.bias"))
        put(self.cls_token, take(e + "cls_token").reshape(-1))
        put(self.pos_embed, take(e + "position_embeddings").reshape(-1, c.hidden_size))
        for i, b in enumerate(self.blocks):
            p = f"{tower}encoder.layer.{i}."
            put(b.qkv.weight, torch.cat([take(p + f"attention.{n}_proj.weight") for n in "qkv"], 0))
            if c.attention_bias:
                put(b.qkv.bias, torch.cat([take(p + f"attention.{n}_proj.bias") for n in "qkv"], 0))
            put(b.proj.weight, take(p + "attention.projection_layer.weight"))
            put(b.proj.bias, take(p + "attention.projection_layer.bias"))
            if c.use_qk_norm:
                put(b.q_norm.weight, take(p + "attention.q_norm.weight"))
                put(b.k_norm.weight, take(p + "attention.k_norm.weight"))
            for norm, name in ((b.norm1, "layernorm_before"), (b.norm2, "layernorm_after")):
                put(norm.weight, take(p + name + ".weight"))
                if norm.bias is not None:
                    put(norm.bias, take(p + name + ".bias"))
            put(b.lambda_1, take(p + "lambda_1"))
            put(b.lambda_2, take(p + "lambda_2"))
            for lin, name in ((b.fc1, "mlp.fc1"), (b.fc2, "mlp.fc2")):
                put(lin.weight, take(p + name + ".weight"))
                put(lin.bias, take(p + name + ".bias"))
        if self.norm is not None:
            put(self.norm.weight, take(tower + "layernorm.weight"))
            put(self.norm.bias, take(tower + "layernorm.bias"))
        put(self.proj_norm.weight, take(projector + "layer_norm.weight"))
        put(self.proj_norm.bias, take(projector + "layer_norm.bias"))
        for lin, name in ((self.proj_fc1, "linear_1"), (self.proj_fc2, "linear_2")):
            put(lin.weight, take(projector + name + ".weight"))
            put(lin.bias, take(projector + name + ".bias"))
        return sorted(k for k in sd if k.startswith((tower, projector)) and k not in used)

    @classmethod
    def from_pretrained(cls, model_dir: str, device="cpu", dtype: Optional[str] = None) -> "InternVisionEncoder":
        """Build tower and projector from a Hugging Face-format InternVL checkpoint directory."""
        import json
        import os
        from ..checkpoint.safetensors_io import CheckpointReader
        with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
            hf = json.load(f)
        cfg = InternVisionConfig.from_hf(hf)
        cfg.dtype = dtype or str(hf.get("torch_dtype", hf.get("dtype", "bfloat16"))).replace("torch.", "")
        enc = cls(cfg)
        reader = CheckpointReader(model_dir)
        keys = list(reader.keys())
        lead = "model." if any(k.startswith("model.vision_tower.") for k in keys) else ""
        names = [k for k in keys if k.startswith((lead + "vision_tower.", lead + "multi_modal_projector."))]
        if not names:
            raise ValueError(f"{model_dir} holds no vision_tower.* tensors")
        left = enc.load_hf_state_dict({k: reader.get(k) for k in names}, lead + "vision_tower.", lead + "multi_modal_projector.")
        if left:
            raise ValueError(f"unused vision tensors: {left[:4]}…")
        return enc.to(device)

    @torch.no_grad()
    def random_init(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator().manual_seed(seed)
        for name, p in self.named_parameters():
            if (name.endswith("weight") and p.dim() == 2) or name in ("pos_embed", "cls_token"):
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
        if self.patch_pad:
            self.patch_embed.weight[:, self.patch_dim:] = 0
        return self

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        n, ch, hh, ww = pixels.shape
        if (hh, ww) != (c.image_size, c.image_size) or ch != c.num_channels:
            raise ValueError(f"tiles must be {c.num_channels} × {c.image_size} × {c.image_size} (got {tuple(pixels.shape[1:])})")
        dev, g, p = pixels.device, c.grid, c.patch_size
        patches = pixels.reshape(n, ch, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(n * g * g, ch * p * p)
        if self.patch_pad:
            patches = torch.nn.functional.pad(patches, (0, self.patch_pad))
        x = self.patch_embed(patches.to(c.compute_dtype)).reshape(n, g * g, -1)
        x = torch.cat([self.cls_token.expand(n, 1, -1), x], dim=1) + self.pos_embed[None]
        tokens = 1 + g * g
        x = x.reshape(n * tokens, -1).contiguous()
        per = (tokens + self.PAGE - 1) // self.PAGE
        table = torch.arange(n * per, dtype=torch.int32).view(n, per)
        meta = build_step_meta([tokens] * n, [0] * n, table, self.PAGE, device=dev)
        if self._kv is None or self._kv.shape[0] < n * per or self._kv.device != dev:
            self._kv = torch.zeros(n * per, 2, c.num_attention_heads, self.PAGE, c.head_dim, dtype=c.compute_dtype, device=dev)
        no_rope = torch.zeros(tokens, 0, dtype=torch.float32, device=dev)          # rotary width 0: keys are stored as they are
        for blk in self.blocks:
            x = blk(x, meta, self._kv, no_rope)
        if self.norm is not None:
            x = self.norm(x)
        x = x.reshape(n, tokens, -1)[:, 1:, :].reshape(n, g, g, -1)                # drop the class token; [N, rows, columns, H]
        # pixel shuffle: fold neighbouring columns, then neighbouring rows, into the channel dimension
        s = c.downsample_ratio
        x = x.reshape(n, g, int(g * s), int(x.shape[-1] / s)).permute(0, 2, 1, 3).contiguous()
        x = x.reshape(n, int(g * s), int(g * s), int(x.shape[-1] / s)).permute(0, 2, 1, 3).contiguous()
        x = x.reshape(n * int(g * s) ** 2, -1)
        return self.proj_fc2(ops.gelu(self.proj_fc1(self.proj_norm(x))))
