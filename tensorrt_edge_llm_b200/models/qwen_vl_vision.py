"""Qwen2-VL / Qwen2.5-VL / Qwen3-VL vision transformer: variable image grids, 2-D rotary positions, window attention, patch
merger, interpolated position table and deepstack taps (Qwen3-VL).

Input is the image processor's patch matrix ``[S, C · T_p · P · P]`` (patches of all images and video frames back to
back, each image in ``merge × merge`` block order) plus one ``(t, h, w)`` grid per image.  The encoder

* embeds patches with one GEMM (the checkpoint's Conv3d has kernel = stride, so it is a linear map of the flat patch),
* gives every patch a rotary table row built from its (row, column) in the image: the first half of the rotary pairs
  turns with the row index, the second half with the column index (``ops.rope_kv_write`` reads per-row tables),
* Qwen2.5-VL: reorders the ``merge²`` blocks window by window, so that a window-attention layer is a ragged step whose
  "sequences" are the windows and a full-attention layer one whose sequences are the frames — both run the paged
  tile attention kernel with the causal mask off — and undoes the order after the merger,
* merges ``merge²`` neighbouring patches into one language-model token (norm → two-layer MLP).

Head dimensions the attention kernel has no tile shape for (80 in the released checkpoints) are zero-padded to 128 in
the weights at load time, each half of the head on its own so that rotate-half pairs stay half a head apart: zero key
features add nothing to the scores, zero value features meet zero projection columns, the padding pairs rotate by
angle zero, so the result is exact while the softmax scale stays ``true_head_dim ** -0.5``.

Parity: ``tensorrt_edgellm/models/qwen2_5_vl`` / ``qwen2_vl`` visual towers with ``vit_attention_plugin``
(``tensorrt_edgellm/models/ops.py:406``) and ``cpp/multimodal/qwenViTRunner.cpp`` (window index, cumulative sequence
lengths, rotary table on the host); the numerical oracle in the tests is the Hugging Face implementation."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
from torch import nn

from .. import ops
from ..ops.meta import build_step_meta


@dataclass
class QwenVisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 3584
    window_size: int = 112                                   # pixels; 0 = every layer attends within the whole frame (Qwen2-VL)
    fullatt_block_indexes: List[int] = field(default_factory=lambda: [7, 15, 23, 31])
    gated_mlp: bool = True                                   # Qwen2.5-VL: SiLU-gated MLP + RMSNorm; Qwen2-VL: quick-GELU MLP + LayerNorm
    eps: float = 1e-6
    rope_theta: float = 10000.0
    dtype: str = "bfloat16"
    # Qwen3-VL: tanh-GELU MLP, biased patch embedding, a learned position table (a square grid, interpolated bilinearly to
    # each image's grid) next to the rotary positions, and "deepstack" mergers that tap the listed blocks
    mlp_act: str = ""                                        # "" = by gated_mlp (swiglu / quick_gelu); "gelu_tanh"
    patch_bias: bool = False
    num_position_embeddings: int = 0
    deepstack_visual_indexes: List[int] = field(default_factory=list)

    @classmethod
    def from_hf(cls, v: Dict) -> "QwenVisionConfig":
        """``vision_config`` of a Qwen2-VL (``embed_dim`` / ``mlp_ratio``), Qwen2.5-VL (``intermediate_size`` / windows) or Qwen3-VL
        (``num_position_embeddings`` / ``deepstack_visual_indexes``) checkpoint."""
        if "num_position_embeddings" in v or "deepstack_visual_indexes" in v:         # Qwen3-VL
            return cls(depth=int(v["depth"]), hidden_size=int(v["hidden_size"]), num_heads=int(v["num_heads"]),
                       intermediate_size=int(v["intermediate_size"]), in_channels=int(v.get("in_channels", 3)),
                       patch_size=int(v.get("patch_size", 16)), temporal_patch_size=int(v.get("temporal_patch_size", 2)),
                       spatial_merge_size=int(v.get("spatial_merge_size", 2)), out_hidden_size=int(v["out_hidden_size"]), window_size=0,
                       fullatt_block_indexes=[], gated_mlp=False, patch_bias=True,
                       mlp_act="gelu_tanh" if "tanh" in str(v.get("hidden_act", "gelu_pytorch_tanh")) else "gelu",
                       num_position_embeddings=int(v.get("num_position_embeddings", 2304)),
                       deepstack_visual_indexes=list(v.get("deepstack_visual_indexes", [8, 16, 24])))
        if "embed_dim" in v:                                 # Qwen2-VL
            h = int(v["embed_dim"])
            return cls(depth=int(v["depth"]), hidden_size=h, num_heads=int(v["num_heads"]), intermediate_size=int(h * v.get("mlp_ratio", 4)),
                       in_channels=int(v.get("in_channels", v.get("in_chans", 3))), patch_size=int(v.get("patch_size", 14)),
                       temporal_patch_size=int(v.get("temporal_patch_size", 2)), spatial_merge_size=int(v.get("spatial_merge_size", 2)),
                       out_hidden_size=int(v["hidden_size"]), window_size=0, fullatt_block_indexes=[], gated_mlp=False)
        return cls(depth=int(v["depth"]), hidden_size=int(v["hidden_size"]), num_heads=int(v["num_heads"]),
                   intermediate_size=int(v["intermediate_size"]), in_channels=int(v.get("in_channels", v.get("in_chans", 3))),
                   patch_size=int(v.get("patch_size", 14)), temporal_patch_size=int(v.get("temporal_patch_size", 2)),
                   spatial_merge_size=int(v.get("spatial_merge_size", 2)), out_hidden_size=int(v["out_hidden_size"]),
                   window_size=int(v.get("window_size", 112)), fullatt_block_indexes=list(v.get("fullatt_block_indexes", [7, 15, 23, 31])))

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def padded_head_dim(self) -> int:
        d = self.head_dim
        if d > 128:
            raise ValueError("vision head dimensions above 128 are not supported")
        return 64 if d <= 64 else 128

    @property
    def compute_dtype(self) -> torch.dtype:
        return {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[self.dtype]

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size ** 2


# ---- host-side index math ----------------------------------------------------------------------------------------

def rotary_rows(grids: Sequence[Sequence[int]], head_dim: int, merge: int, theta: float = 10000.0) -> torch.Tensor:
    """Per-patch rotary table ``[S, head_dim]`` (cos half | sin half) for patches in ``merge × merge`` block order:
    pairs ``0 .. head_dim/4 - 1`` use the patch's row, the rest its column."""
    quarter = head_dim // 4
    inv = 1.0 / (theta ** (torch.arange(0, quarter, dtype=torch.float64) * 2.0 / (head_dim // 2)))
    rows = []
    for t, h, w in grids:
        hp = torch.arange(h)[:, None].expand(h, w).reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).reshape(-1)
        wp = torch.arange(w)[None, :].expand(h, w).reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).reshape(-1)
        ang = torch.cat([hp[:, None].double() * inv[None, :], wp[:, None].double() * inv[None, :]], dim=1)      # [h·w, head_dim/2]
        rows.append(torch.cat([ang.cos(), ang.sin()], dim=1).repeat(int(t), 1))
    return torch.cat(rows, dim=0).float()


def window_order(grids: Sequence[Sequence[int]], window_size: int, merge: int, patch: int) -> Tuple[torch.Tensor, List[int]]:
    """Order of the merged ``merge × merge`` units that makes every attention window contiguous, and the window lengths in
    patches.  A window covers ``window_size`` pixels per side; windows at the right and bottom edges are smaller."""
    unit = window_size // merge // patch
    if unit <= 0:
        raise ValueError("window_size must cover at least one merged patch")
    order, lengths, base = [], [], 0
    for t, h, w in grids:
        gh, gw = h // merge, w // merge
        idx = torch.arange(int(t) * gh * gw).reshape(int(t), gh, gw)
        for f in range(int(t)):
            for y0 in range(0, gh, unit):
                for x0 in range(0, gw, unit):
                    win = idx[f, y0:y0 + unit, x0:x0 + unit].reshape(-1)
                    order.append(win + base)
                    lengths.append(int(win.numel()) * merge * merge)
        base += int(t) * gh * gw
    return torch.cat(order), lengths


# ---- modules -----------------------------------------------------------------------------------------------------

class _Lin(nn.Module):
    def __init__(self, i, o, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(o, i, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype), requires_grad=False)

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class _Norm(nn.Module):
    def __init__(self, dim, eps, dtype, rms: bool):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.bias = None if rms else nn.Parameter(torch.zeros(dim, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps) if self.bias is None else ops.layernorm(x, self.weight, self.bias, self.eps)


class QwenVisionBlock(nn.Module):
    def __init__(self, cfg: QwenVisionConfig):
        super().__init__()
        dt, h, hp = cfg.compute_dtype, cfg.hidden_size, cfg.num_heads * cfg.padded_head_dim
        self.cfg = cfg
        self.norm1, self.norm2 = _Norm(h, cfg.eps, dt, cfg.gated_mlp), _Norm(h, cfg.eps, dt, cfg.gated_mlp)
        self.qkv, self.proj = _Lin(h, 3 * hp, dt), _Lin(hp, h, dt)
        self.fc1 = _Lin(h, cfg.intermediate_size * (2 if cfg.gated_mlp else 1), dt)      # gated: rows are [gate | up]
        self.fc2 = _Lin(cfg.intermediate_size, h, dt)

    def forward(self, x, meta, kv, table):
        c = self.cfg
        qkv = self.qkv(self.norm1(x))
        q = ops.rope_kv_write(qkv, kv, meta, table, c.num_heads, c.num_heads, c.padded_head_dim)
        a = ops.paged_attention(q, kv, meta, c.head_dim ** -0.5, causal=False)
        x = x + self.proj(a.reshape(a.shape[0], -1))
        y = self.fc1(self.norm2(x))
        if c.gated_mlp:
            y = ops.swiglu(y)
        elif c.mlp_act in ("gelu_tanh", "gelu"):
            y = ops.gelu(y, c.mlp_act == "gelu_tanh")
        else:
            y = (y.float() * torch.sigmoid(1.702 * y.float())).to(y.dtype)               # quick GELU
        return x + self.fc2(y)


class _DeepstackMerger(nn.Module):
    def __init__(self, cfg: QwenVisionConfig):
        super().__init__()
        wide = cfg.hidden_size * cfg.spatial_merge_size ** 2
        self.norm = _Norm(wide, 1e-6, cfg.compute_dtype, False)
        self.fc1, self.fc2 = _Lin(wide, wide, cfg.compute_dtype), _Lin(wide, cfg.out_hidden_size, cfg.compute_dtype)

    def forward(self, x):
        return self.fc2(ops.gelu(self.fc1(self.norm(x.reshape(-1, self.norm.weight.shape[0]).contiguous()))))


def interpolated_positions(table: torch.Tensor, grids: Sequence[Sequence[int]], merge: int) -> torch.Tensor:
    """Rows of the learned ``side × side`` position table resampled bilinearly (corners aligned) to every image's
    ``h × w`` grid, repeated per frame and laid out in ``merge × merge`` block order: ``[S, H]``."""
    side = int(round(table.shape[0] ** 0.5))
    out = []
    for t, h, w in grids:
        ys, xs = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
        y0, x0 = ys.int(), xs.int()
        y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
        dy, dx = (ys - y0)[:, None], (xs - x0)[None, :]
        tb = table.float()
        g = lambda yy, xx: tb[(yy[:, None] * side + xx[None, :]).long().reshape(-1).to(table.device)].reshape(h, w, -1)
        wgt = lambda a: a.to(table.device)[..., None]
        p = (g(y0, x0) * wgt((1 - dy) * (1 - dx)) + g(y0, x1) * wgt((1 - dy) * dx) + g(y1, x0) * wgt(dy * (1 - dx)) + g(y1, x1) * wgt(dy * dx))
        p = p.reshape(h // merge, merge, w // merge, merge, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
        out.append(p.repeat(int(t), 1))
    return torch.cat(out, 0).to(table.dtype)


class QwenVisionEncoder(nn.Module):
    """``forward(patches [S, patch_dim], grids [(t, h, w), …])`` → ``[S / merge², out_hidden_size]`` rows in image order."""

    PAGE = 64

    def __init__(self, cfg: QwenVisionConfig):
        super().__init__()
        self.cfg = cfg
        dt, h = cfg.compute_dtype, cfg.hidden_size
        self.patch_embed = _Lin(cfg.patch_dim, h, dt)
        if not cfg.patch_bias:
            self.patch_embed.bias = None                     # Qwen2 / 2.5: the checkpoint's Conv3d has no bias
        self.pos_embed = (nn.Parameter(torch.zeros(cfg.num_position_embeddings, h, dtype=dt), requires_grad=False)
                          if cfg.num_position_embeddings else None)
        self.blocks = nn.ModuleList([QwenVisionBlock(cfg) for _ in range(cfg.depth)])
        m2 = cfg.spatial_merge_size ** 2
        self.ln_q = _Norm(h, 1e-6, dt, cfg.gated_mlp)
        self.merger_fc1, self.merger_fc2 = _Lin(h * m2, h * m2, dt), _Lin(h * m2, cfg.out_hidden_size, dt)
        # deepstack: merged features of intermediate blocks (norm over the merged row, then the same two-layer shape)
        self.deepstack = nn.ModuleList([_DeepstackMerger(cfg) for _ in cfg.deepstack_visual_indexes])
        self._kv: Optional[torch.Tensor] = None

    # ---- weights ---------------------------------------------------------------------------------
    def _pad_heads(self, w: torch.Tensor, axis: int) -> torch.Tensor:
        """Zero-pad every head's slice of ``w`` from ``head_dim`` to ``padded_head_dim`` along ``axis``.  Each half of the
        head is padded on its own (``[first half | 0 | second half | 0]``), so the rotate-half partner of feature ``j``
        stays at ``j + padded_head_dim / 2`` and the full-width rotary kernels apply."""
        c = self.cfg
        d, dp = c.head_dim, c.padded_head_dim
        if d == dp:
            return w
        shape = list(w.shape)
        groups = shape[axis] // d
        w = w.reshape(shape[:axis] + [groups, 2, d // 2] + shape[axis + 1:])
        pad = torch.zeros(shape[:axis] + [groups, 2, (dp - d) // 2] + shape[axis + 1:], dtype=w.dtype, device=w.device)
        return torch.cat([w, pad], dim=axis + 2).reshape(shape[:axis] + [groups * dp] + shape[axis + 1:])

    def _pad_table(self, table: torch.Tensor) -> torch.Tensor:
        """Rotary rows for the padded head: the padding pairs get angle zero (cos 1, sin 0)."""
        c = self.cfg
        half, extra = c.head_dim // 2, (c.padded_head_dim - c.head_dim) // 2
        if extra == 0:
            return table
        rows = table.shape[0]
        return torch.cat([table[:, :half], torch.ones(rows, extra), table[:, half:], torch.zeros(rows, extra)], dim=1)

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], prefix: str = "visual.") -> List[str]:
        """Fill the encoder from Hugging Face tensors (names under ``prefix``); returns the names it did not use."""
        c = self.cfg
        sd = {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}
        used = set()

        def take(name):
            used.add(name)
            return sd[name]

        def put(param, value):
            if tuple(param.shape) != tuple(value.shape):
                raise ValueError(f"shape {tuple(value.shape)} does not fit {tuple(param.shape)}")
            param.copy_(value.to(param.dtype))
        put(self.patch_embed.weight, take("patch_embed.proj.weight").reshape(c.hidden_size, -1))
        if c.patch_bias:
            put(self.patch_embed.bias, take("patch_embed.proj.bias"))
        if self.pos_embed is not None:
            put(self.pos_embed, take("pos_embed.weight"))
        q3 = bool(c.num_position_embeddings)                 # Qwen3-VL tensor names
        for i, b in enumerate(self.blocks):
            p = f"blocks.{i}."
            for norm, name in ((b.norm1, "norm1"), (b.norm2, "norm2")):
                put(norm.weight, take(p + name + ".weight"))
                if norm.bias is not None:
                    put(norm.bias, take(p + name + ".bias"))
            put(b.qkv.weight, self._pad_heads(take(p + "attn.qkv.weight"), 0))
            put(b.qkv.bias, self._pad_heads(take(p + "attn.qkv.bias"), 0))
            put(b.proj.weight, self._pad_heads(take(p + "attn.proj.weight"), 1))
            put(b.proj.bias, take(p + "attn.proj.bias"))
            if c.gated_mlp:
                put(b.fc1.weight, torch.cat([take(p + "mlp.gate_proj.weight"), take(p + "mlp.up_proj.weight")], 0))
                put(b.fc1.bias, torch.cat([take(p + "mlp.gate_proj.bias"), take(p + "mlp.up_proj.bias")], 0))
                put(b.fc2.weight, take(p + "mlp.down_proj.weight"))
                put(b.fc2.bias, take(p + "mlp.down_proj.bias"))
            else:
                for lin, name in ((b.fc1, "mlp.linear_fc1" if q3 else "mlp.fc1"), (b.fc2, "mlp.linear_fc2" if q3 else "mlp.fc2")):
                    put(lin.weight, take(p + name + ".weight"))
                    put(lin.bias, take(p + name + ".bias"))
        ln = "merger.norm" if q3 else "merger.ln_q"
        put(self.ln_q.weight, take(ln + ".weight"))
        if self.ln_q.bias is not None:
            put(self.ln_q.bias, take(ln + ".bias"))
        for lin, name in ((self.merger_fc1, "merger.linear_fc1" if q3 else "merger.mlp.0"), (self.merger_fc2, "merger.linear_fc2" if q3 else "merger.mlp.2")):
            put(lin.weight, take(name + ".weight"))
            put(lin.bias, take(name + ".bias"))
        for k, dm in enumerate(self.deepstack):
            p = f"deepstack_merger_list.{k}."
            put(dm.norm.weight, take(p + "norm.weight"))
            put(dm.norm.bias, take(p + "norm.bias"))
            for lin, name in ((dm.fc1, "linear_fc1"), (dm.fc2, "linear_fc2")):
                put(lin.weight, take(p + name + ".weight"))
                put(lin.bias, take(p + name + ".bias"))
        return sorted(set(sd) - used)

    @classmethod
    def from_pretrained(cls, model_dir: str, device="cpu", dtype: Optional[str] = None) -> "QwenVisionEncoder":
        """Build the tower from a Qwen2-VL / Qwen2.5-VL checkpoint directory (``vision_config`` of ``config.json``, tensors
        named ``visual.*`` or ``model.visual.*`` in its safetensors files)."""
        import json
        import os
        from ..checkpoint.safetensors_io import CheckpointReader
        with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
            hf = json.load(f)
        if "vision_config" not in hf:
            raise ValueError(f"{model_dir} has no vision_config")
        cfg = QwenVisionConfig.from_hf(hf["vision_config"])
        cfg.dtype = dtype or str(hf.get("torch_dtype", hf.get("dtype", "bfloat16"))).replace("torch.", "")
        enc = cls(cfg)
        reader = CheckpointReader(model_dir)
        names = [k for k in reader.keys() if k.startswith(("visual.", "model.visual."))]
        if not names:
            raise ValueError(f"{model_dir} holds no visual.* tensors")
        prefix = "model.visual." if names[0].startswith("model.") else "visual."
        left = enc.load_hf_state_dict({k: reader.get(k) for k in names}, prefix=prefix)
        if left:
            raise ValueError(f"unused vision tensors: {left[:4]}…")
        return enc.to(device)

    # ---- forward ---------------------------------------------------------------------------------
    def _meta(self, lengths: Sequence[int], device):
        pages = [(n + self.PAGE - 1) // self.PAGE for n in lengths]
        table = torch.full((len(lengths), max(pages)), -1, dtype=torch.int32)
        at = 0
        for i, n in enumerate(pages):
            table[i, :n] = torch.arange(at, at + n, dtype=torch.int32)
            at += n
        return build_step_meta(list(lengths), [0] * len(lengths), table, self.PAGE, device=device), at

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grids: Sequence[Sequence[int]], return_deepstack: bool = False):
        """``return_deepstack``: also return the list of deepstack features (one ``[S / merge², out_hidden]`` tensor per tapped
        block, in the order of ``deepstack_visual_indexes``)."""
        c = self.cfg
        m2 = c.spatial_merge_size ** 2
        dev = patches.device
        grids = [tuple(int(v) for v in g) for g in grids]
        total = sum(t * h * w for t, h, w in grids)
        if patches.shape[0] != total or patches.shape[1] != c.patch_dim:
            raise ValueError(f"patch matrix {tuple(patches.shape)} does not fit grids {grids} (want [{total}, {c.patch_dim}])")
        if any(h % c.spatial_merge_size or w % c.spatial_merge_size for _, h, w in grids):
            raise ValueError("grid heights and widths must be multiples of the spatial merge size")
        x = ops.linear(patches.to(c.compute_dtype), self.patch_embed.weight, self.patch_embed.bias)
        if self.pos_embed is not None:
            x = x + interpolated_positions(self.pos_embed, grids, c.spatial_merge_size).to(x.dtype)
        table = self._pad_table(rotary_rows(grids, c.head_dim, c.spatial_merge_size, c.rope_theta)).to(dev)
        frame_meta, frame_pages = self._meta([h * w for t, h, w in grids for _ in range(t)], dev)
        win_meta, win_pages, order = None, 0, None
        if c.window_size > 0:
            order, win_lengths = window_order(grids, c.window_size, c.spatial_merge_size, c.patch_size)
            order = order.to(dev)
            x = x.reshape(total // m2, m2, -1)[order].reshape(total, -1)
            table = table.reshape(total // m2, m2, -1)[order].reshape(total, -1)
            win_meta, win_pages = self._meta(win_lengths, dev)
        pages = max(frame_pages, win_pages)
        if self._kv is None or self._kv.shape[0] < pages or self._kv.device != dev:
            self._kv = torch.zeros(pages, 2, c.num_heads, self.PAGE, c.padded_head_dim, dtype=c.compute_dtype, device=dev)
        rows = torch.arange(total, dtype=torch.int32, device=dev)
        for meta in (frame_meta, win_meta):
            if meta is not None:
                meta.rope_rows, meta.rope_pos = table.contiguous(), rows       # every patch reads its own table row
        taps = []
        for i, blk in enumerate(self.blocks):
            full = win_meta is None or i in c.fullatt_block_indexes
            x = blk(x, frame_meta if full else win_meta, self._kv, table)
            if i in c.deepstack_visual_indexes:
                taps.append(self.deepstack[c.deepstack_visual_indexes.index(i)](x))
        x = self.ln_q(x).reshape(total // m2, m2 * c.hidden_size)
        y = self.merger_fc2(ops.gelu(self.merger_fc1(x.contiguous())))
        if order is not None:
            y = y[torch.argsort(order)]
        return (y, taps) if return_deepstack else y

    @torch.no_grad()
    def random_init(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator().manual_seed(seed)
        for name, p in self.named_parameters():
            if (name.endswith("weight") and p.dim() == 2) or name == "pos_embed":
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
        d, dp = self.cfg.head_dim, self.cfg.padded_head_dim
        if d != dp:                                           # keep the padding features zero for random weights too
            live = torch.zeros(dp, dtype=torch.bool)
            live[:d // 2] = True
            live[dp // 2:dp // 2 + d // 2] = True
            for b in self.blocks:
                b.qkv.weight.view(-1, dp, b.qkv.weight.shape[1])[:, ~live, :] = 0
                b.proj.weight.view(b.proj.weight.shape[0], -1, dp)[:, :, ~live] = 0
        return self


def patchify_frames(frames: torch.Tensor, cfg: QwenVisionConfig) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """``frames [F, C, H, W]`` (normalised pixels; a still image is one frame, repeated to fill a temporal patch) →
    the processor's patch matrix ``[t · h · w, C · T_p · P · P]`` in ``merge × merge`` block order and its ``(t, h, w)`` grid."""
    f, ch, hh, ww = frames.shape
    tp, p, m = cfg.temporal_patch_size, cfg.patch_size, cfg.spatial_merge_size
    if f % tp:
        frames = torch.cat([frames, frames[-1:].expand(tp - f % tp, -1, -1, -1)], dim=0)
        f = frames.shape[0]
    if hh % (p * m) or ww % (p * m):
        raise ValueError(f"image sides must be multiples of {p * m} (patch × merge); resize first (smart_resize)")
    t, h, w = f // tp, hh // p, ww // p
    x = frames.reshape(t, tp, ch, h // m, m, p, w // m, m, p).permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return x.reshape(t * h * w, ch * tp * p * p).contiguous(), (t, h, w)
