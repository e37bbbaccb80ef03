"""Vision transformer encoder + projector producing embeddings for the language model.

Pre-LayerNorm ViT blocks (learned position embeddings, bidirectional attention, GELU MLP) over image patches,
followed by an optional ``merge × merge`` spatial merge and a two-layer projector into the LLM's hidden size —
the common shape of the InternViT / CLIP / Qwen-VL style encoders.  The attention runs the same paged tile kernel
as the decoder with the causal mask switched off (``ops.paged_attention(..., causal=False)``): an image is one
"sequence" whose patches are written to a scratch KV pool and attended in full.

Parity: the visual encoders of ``tensorrt_edgellm/models/*vl*`` with ``vit_attention_plugin``
(``tensorrt_edgellm/models/ops.py:406``) and the runner contract of ``cpp/multimodal/`` (image → embedding rows that
replace the image-token rows of the prompt)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
from torch import nn

from .. import ops
from ..ops.meta import build_step_meta


@dataclass
class VisionConfig:
    hidden_size: int = 1024
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    intermediate_size: int = 4096
    patch_size: int = 14
    image_size: int = 448
    in_channels: int = 3
    layer_norm_eps: float = 1e-6
    spatial_merge: int = 2                 # merge x merge neighbouring patches become one LLM token
    out_hidden_size: int = 4096            # the language model's hidden size
    gelu_tanh: bool = False
    dtype: str = "bfloat16"

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def grid(self) -> int:
        return self.image_size // self.patch_size

    @property
    def compute_dtype(self) -> torch.dtype:
        return getattr(torch, self.dtype)


class _LayerNorm(nn.Module):
    def __init__(self, dim, eps, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        return ops.layernorm(x, self.weight, self.bias, self.eps)


class _Linear(nn.Module):
    def __init__(self, i, o, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(o, i, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype), requires_grad=False)

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class VitBlock(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        dt, h = cfg.compute_dtype, cfg.hidden_size
        self.cfg = cfg
        self.norm1, self.norm2 = _LayerNorm(h, cfg.layer_norm_eps, dt), _LayerNorm(h, cfg.layer_norm_eps, dt)
        self.qkv, self.proj = _Linear(h, 3 * h, dt), _Linear(h, h, dt)
        self.fc1, self.fc2 = _Linear(h, cfg.intermediate_size, dt), _Linear(cfg.intermediate_size, h, dt)

    def forward(self, x, meta, kv_layer, no_rope):
        c = self.cfg
        qkv = self.qkv(self.norm1(x))
        q = ops.rope_kv_write(qkv, kv_layer, meta, no_rope, c.num_attention_heads, c.num_attention_heads, c.head_dim)
        a = ops.paged_attention(q, kv_layer, meta, c.head_dim ** -0.5, causal=False)
        x = x + self.proj(a.reshape(a.shape[0], -1))
        return x + self.fc2(ops.gelu(self.fc1(self.norm2(x)), c.gelu_tanh))


class VisionEncoder(nn.Module):
    """``forward(patches [N_img, grid², C·P·P])`` → ``[N_img · (grid / merge)², out_hidden]`` embedding rows."""

    def __init__(self, cfg: VisionConfig):
        super().__init__()
        if cfg.head_dim not in (64, 128):
            raise ValueError("the attention kernel takes head dimensions of 64 or 128")
        if cfg.grid % cfg.spatial_merge:
            raise ValueError("the patch grid must be divisible by the spatial merge factor")
        self.cfg = cfg
        dt, h = cfg.compute_dtype, cfg.hidden_size
        self.patch_embed = _Linear(cfg.in_channels * cfg.patch_size ** 2, h, dt)
        self.pos_embed = nn.Parameter(torch.zeros(cfg.grid ** 2, h, dtype=dt), requires_grad=False)
        self.blocks = nn.ModuleList([VitBlock(cfg) for _ in range(cfg.num_hidden_layers)])
        self.norm = _LayerNorm(h, cfg.layer_norm_eps, dt)
        m2 = cfg.spatial_merge ** 2
        self.merger_fc1, self.merger_fc2 = _Linear(h * m2, h * m2, dt), _Linear(h * m2, cfg.out_hidden_size, dt)
        self._kv: Optional[torch.Tensor] = None

    @torch.no_grad()
    def random_init(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator().manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("weight") and p.dim() == 2 or name == "pos_embed":
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
        return self

    @staticmethod
    def patchify(images: torch.Tensor, patch: int) -> torch.Tensor:
        """``[N, C, H, W]`` pixels → ``[N, (H/P)(W/P), C·P·P]`` row-major patches."""
        n, c, hh, ww = images.shape
        x = images.reshape(n, c, hh // patch, patch, ww // patch, patch).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(n, (hh // patch) * (ww // patch), c * patch * patch)

    def _scratch_kv(self, n_img: int, tokens: int, device) -> torch.Tensor:
        page = 64
        pages = n_img * ((tokens + page - 1) // page)
        c = self.cfg
        if self._kv is None or self._kv.shape[0] < pages or self._kv.device != device:
            self._kv = torch.zeros(pages, 2, c.num_attention_heads, page, c.head_dim, dtype=c.compute_dtype, device=device)
        return self._kv

    def forward(self, patches: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        n_img, tokens, _ = patches.shape
        dev = patches.device
        x = self.patch_embed(patches.reshape(n_img * tokens, -1).to(c.compute_dtype)) + self.pos_embed[:tokens].repeat(n_img, 1)
        page = 64
        per = (tokens + page - 1) // page
        table = torch.arange(n_img * per, dtype=torch.int32).view(n_img, per)
        meta = build_step_meta([tokens] * n_img, [0] * n_img, table, page, device=dev)
        kv = self._scratch_kv(n_img, tokens, dev)
        no_rope = torch.zeros(tokens, 0, dtype=torch.float32, device=dev)          # rotary width 0: keys are stored as they are
        for blk in self.blocks:
            x = blk(x, meta, kv, no_rope)
        x = self.norm(x)
        m, g = c.spatial_merge, int(round(tokens ** 0.5))
        x = x.view(n_img, g // m, m, g // m, m, c.hidden_size).permute(0, 1, 3, 2, 4, 5).reshape(n_img * (g // m) ** 2, m * m * c.hidden_size)
        return self.merger_fc2(ops.gelu(self.merger_fc1(x.contiguous()), c.gelu_tanh))


def merge_image_embeddings(token_ids: Sequence[int], text_embeds: torch.Tensor, image_embeds: torch.Tensor, image_token_id: int
                           ) -> torch.Tensor:
    """Replace the rows of ``text_embeds`` at ``image_token_id`` positions by the image embedding rows, in order."""
    ids = torch.as_tensor(list(token_ids), device=text_embeds.device)
    pos = (ids == image_token_id).nonzero(as_tuple=True)[0]
    if pos.numel() != image_embeds.shape[0]:
        raise ValueError(f"prompt has {pos.numel()} image tokens but the encoder produced {image_embeds.shape[0]} rows")
    out = text_embeds.clone()
    out[pos] = image_embeds.to(out.dtype)
    return out


class EncoderCache:
    """Encoder outputs keyed by a hash of the decoded media bytes, least-recently-used within a byte budget
    (``--encoder-cache-budget-bytes`` in the reference, ``docs/source/user_guide/features/kv-cache-reuse.md:166-188``):
    the same image or clip in a later request skips the encoder."""

    def __init__(self, budget_bytes: int):
        from collections import OrderedDict
        self.budget, self.used = int(budget_bytes), 0
        self._items: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        self.hits = self.misses = 0

    @staticmethod
    def key(data) -> str:
        import hashlib
        if isinstance(data, torch.Tensor):
            t = data.detach().contiguous().cpu()
            data = t.view(torch.uint8).numpy().tobytes() + str((tuple(t.shape), t.dtype)).encode()
        return hashlib.blake2b(bytes(data), digest_size=16).hexdigest()

    def get(self, key: str) -> Optional[torch.Tensor]:
        v = self._items.get(key)
        if v is None:
            self.misses += 1
            return None
        self._items.move_to_end(key)
        self.hits += 1
        return v

    def put(self, key: str, value: torch.Tensor) -> None:
        size = value.numel() * value.element_size()
        if size > self.budget or key in self._items:
            return
        while self.used + size > self.budget and self._items:
            _, old = self._items.popitem(last=False)
            self.used -= old.numel() * old.element_size()
        self._items[key] = value
        self.used += size

    def encode(self, encoder, inputs: torch.Tensor) -> torch.Tensor:
        """Run ``encoder`` on the items of ``inputs`` (first dimension) that are not cached; rows come back in input order."""
        keys = [self.key(x) for x in inputs]
        outs: List[Optional[torch.Tensor]] = [self.get(k) for k in keys]
        todo = [i for i, o in enumerate(outs) if o is None]
        if todo:
            fresh = encoder(inputs[todo])
            per = fresh.shape[0] // len(todo)
            for j, i in enumerate(todo):
                outs[i] = fresh[j * per:(j + 1) * per]
                self.put(keys[i], outs[i])
        return torch.cat(outs, 0)


def encode_data_parallel(encoder, inputs: torch.Tensor, comm) -> torch.Tensor:
    """Vision / audio data parallelism over the tensor-parallel ranks: every rank encodes a contiguous shard of the
    items and the embedding rows are all-gathered, so each rank ends with all rows in input order
    (``cpp/runtime/visionDataParallel/visionGather.*`` and ``cpp/runtime/multiDevice/runtimeCoordinator.cpp:376-392``).
    The item count is padded to a multiple of the world size (the padding items repeat the last one and are dropped)."""
    world, rank = comm.world_size, comm.rank
    n = inputs.shape[0]
    if world == 1 or n == 0:
        return encoder(inputs)
    per = (n + world - 1) // world
    idx = torch.arange(rank * per, (rank + 1) * per).clamp(max=n - 1)
    mine = encoder(inputs[idx])                                   # [per · rows_per_item, H]
    full = comm.all_gather_rows(mine.contiguous())                # rank-major = input order
    rows_per_item = mine.shape[0] // per
    return full[:n * rows_per_item]


def dart_prune(embeds: torch.Tensor, keep: int, num_pivots: int = 8) -> torch.Tensor:
    """Duplication-aware visual-token pruning (the DART pruner of ``cpp/runtime/preprocess/`` / ``cpp/kernels/dart`` in
    the reference): a few pivot rows are chosen — those with the largest norm, spread over the image — and the rows most
    similar (cosine) to any pivot are dropped as duplicates until ``keep`` rows remain.  Returns the sorted indices of
    the rows to keep; pivots always survive."""
    n = embeds.shape[0]
    if keep >= n:
        return torch.arange(n, device=embeds.device)
    x = torch.nn.functional.normalize(embeds.float(), dim=-1)
    num_pivots = max(1, min(num_pivots, keep))
    # one pivot per contiguous stripe of the image (its highest-norm row), so pivots do not cluster in one corner
    norms = embeds.float().norm(dim=-1)
    bounds = torch.linspace(0, n, num_pivots + 1).long()
    pivots = torch.stack([bounds[i] + norms[bounds[i]:bounds[i + 1]].argmax() for i in range(num_pivots) if bounds[i + 1] > bounds[i]])
    sim = (x @ x[pivots].t()).amax(dim=-1)                      # closeness of every row to its nearest pivot
    sim[pivots] = -2.0                                          # pivots are kept unconditionally
    order = sim.argsort()                                       # least redundant first
    return order[:keep].sort().values


def sample_video_frames(num_frames: int, video_fps: float, target_fps: float = 2.0, min_frames: int = 4, max_frames: int = 768,
                        multiple_of: int = 2) -> List[int]:
    """Frame indices to decode from a video (``tensorrt_edgellm/server/media/video_sampling.py``): about ``target_fps``
    frames per second, clamped to ``[min_frames, max_frames]`` and rounded to ``multiple_of`` (temporal patching pairs
    frames), spread evenly over the clip."""
    if num_frames <= 0 or video_fps <= 0:
        raise ValueError("a video needs frames and a frame rate")
    want = num_frames / video_fps * target_fps
    want = min(max(want, min_frames), max_frames, num_frames)
    want = max(multiple_of, int(want // multiple_of) * multiple_of)
    want = min(want, num_frames - num_frames % multiple_of if num_frames >= multiple_of else num_frames)
    if want <= 1:
        return [0]
    return [int(round(i * (num_frames - 1) / (want - 1))) for i in range(want)]
