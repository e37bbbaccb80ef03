"""Plain-PyTorch statements of every operator (fp32 math).

These bodies are (a) the CPU execution path, so the whole runtime steps without a GPU, and
(b) the numerical oracle each CUDA kernel is tested against.  They favour clarity over speed.

Operator semantics follow the reference's CPU statements: RMSNorm
(``tensorrt_edgellm/models/default/modeling_default.py:163-182``), rotate-half RoPE and causal
GQA attention (``unittests/support/references.h:29-65``), NVFP4 math
(``tensorrt_edgellm/models/ops.py:826-909``), MoE routing
(``unittests/support/references.cpp:1384-1476``), Mamba2 state update
(``unittests/cpp/kernels/mamba/mambaSelectiveStateUpdateTests.cu:62-160``), gated delta rule
(``unittests/cpp/kernels/gdnKernels/gdnCuteDslTests.cu:157-238``).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .meta import StepMeta

# ------------------------------------------------------------------------------------------
# norms / activations


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps)
    return (y.to(x.dtype).float() * weight.float()).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``res = x + residual`` (in the activation dtype), ``y = rmsnorm(res)``; returns (y, res)."""
    res = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(res, weight, eps), res


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


def gated_group_rmsnorm(x: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, n_groups: int, eps: float) -> torch.Tensor:
    """Mamba2 output norm: ``g = x * silu(z)``, RMS-normalise each of ``n_groups`` slices, scale."""
    g = x.float() * F.silu(z.float())
    shp = g.shape
    g = g.reshape(*shp[:-1], n_groups, shp[-1] // n_groups)
    g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps)
    return (g.reshape(shp).to(x.dtype).float() * weight.float()).to(x.dtype)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` where the last dim holds ``[gate | up]`` halves."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def relu2(x: torch.Tensor) -> torch.Tensor:
    return F.relu(x.float()).pow(2).to(x.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return table[ids.long()]


# ------------------------------------------------------------------------------------------
# RoPE


def rope_frequencies(max_pos: int, rotary_dim: int, theta: float, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, float]:
    """``(inverse frequencies [rotary_dim / 2] fp64, attention factor)`` of a RoPE table of ``max_pos`` positions.

    Supports the default, ``linear``, ``dynamic`` (NTK, evaluated at the table length), ``llama3``, ``yarn`` and
    ``longrope`` (per-pair short / long factors) frequency scalings — the ``RopeType`` set of
    ``cpp/runtime/llmRuntimeUtils.h`` and ``cpp/kernels/posEncoding/initializeCosSinCache.cu`` in the reference."""
    half = rotary_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / rotary_dim))
    att = 1.0
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        factor = float(scaling.get("factor", 1.0))
        if kind == "linear":
            inv = inv / factor
        elif kind == "dynamic":
            # NTK-aware: once the table is longer than the trained context the base grows so that the longest wavelength
            # still spans it (the table is built once, for `max_pos` positions)
            orig = float(scaling.get("original_max_position_embeddings", max_pos))
            if max_pos > orig:
                base = theta * ((factor * max_pos / orig) - (factor - 1)) ** (rotary_dim / (rotary_dim - 2))
                inv = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / rotary_dim))
        elif kind == "longrope":
            orig = float(scaling.get("original_max_position_embeddings", max_pos))
            ext = torch.tensor(scaling["long_factor"] if max_pos > orig else scaling["short_factor"], dtype=torch.float64)
            if ext.numel() != half:
                raise ValueError(f"longrope factors need {half} entries")
            inv = inv / ext
            ratio = max(float(scaling.get("factor", max_pos / orig)), 1.0)
            att = float(scaling.get("attention_factor") or (1.0 if ratio <= 1.0 else math.sqrt(1 + math.log(ratio) / math.log(orig))))
        elif kind == "llama3":
            lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv
            smooth = ((orig / wavelen) - lo) / (hi - lo)
            scaled = torch.where(wavelen > orig / lo, inv / factor,
                                 torch.where(wavelen < orig / hi, inv, (1 - smooth) * inv / factor + smooth * inv))
            inv = scaled
        elif kind == "yarn":
            orig = float(scaling.get("original_max_position_embeddings", 4096))
            bf, bs = float(scaling.get("beta_fast", 32)), float(scaling.get("beta_slow", 1))

            def corr(rot):
                return rotary_dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(theta))
            lo_i, hi_i = max(math.floor(corr(bf)), 0), min(math.ceil(corr(bs)), half - 1)
            ramp = ((torch.arange(half, dtype=torch.float64) - lo_i) / max(hi_i - lo_i, 1e-3)).clamp(0, 1)
            inv = inv / factor * ramp + inv * (1 - ramp)
            att = float(scaling.get("attention_factor") or (0.1 * math.log(factor) + 1.0))
    return inv, att


def rope_cos_sin(max_pos: int, rotary_dim: int, theta: float, scaling: Optional[dict] = None,
                 device="cpu") -> torch.Tensor:
    """``[max_pos, rotary_dim]`` table: first half cos, second half sin (fp32; angles in fp64), for the frequencies of
    :func:`rope_frequencies`."""
    inv, att = rope_frequencies(max_pos, rotary_dim, theta, scaling)
    pos = torch.arange(max_pos, dtype=torch.float64)
    ang = pos[:, None] * inv[None, :]
    return torch.cat([ang.cos() * att, ang.sin() * att], dim=-1).float().to(device)


def mrope_rows(cos_sin: torch.Tensor, positions3: torch.Tensor, sections: Sequence[int]) -> torch.Tensor:
    """Multimodal RoPE (Qwen2-VL): rotary pair ``i`` takes its angle from the temporal, height or width position
    according to ``sections`` (pairs per component, summing to ``D / 2``).  ``cos_sin [P, D]`` is the ordinary table,
    ``positions3 [3, T]``; returns per-row tables ``[T, D]`` to be looked up with positions ``0..T-1``."""
    half = cos_sin.shape[-1] // 2
    if sum(sections) != half or len(sections) != 3:
        raise ValueError(f"mrope sections {list(sections)} must be three counts summing to {half}")
    comp = torch.repeat_interleave(torch.arange(3, device=cos_sin.device), torch.tensor(list(sections), device=cos_sin.device))
    pos = positions3.long().to(cos_sin.device)[comp]                  # [half, T]: position used by pair i at row t
    cols = torch.arange(half, device=cos_sin.device)[:, None].expand_as(pos)
    cos = cos_sin[pos, cols]                                          # [half, T]
    sin = cos_sin[pos, cols + half]
    return torch.cat([cos.t(), sin.t()], dim=-1).contiguous()


def mrope_positions(token_ids: Sequence[int], image_token_id: int, grids: Sequence[Sequence[int]], spatial_merge: int = 2):
    """3-D positions of a prompt whose images appear as runs of ``image_token_id`` (Qwen2-VL ``get_rope_index``): text rows
    advance all three components together; an image of grid ``(t, h, w)`` patches (``h``, ``w`` before the spatial
    merge) occupies ``t · h/m · w/m`` rows whose components count frames, rows and columns from the current offset,
    and the text after it continues from the largest component plus one.  Returns ``(positions3 [3, T] int32, delta)``
    with ``delta`` = next position − ``T``, the offset decode steps add to the sequence length."""
    ids = list(token_ids)
    out = [[], [], []]
    nxt, i, img = 0, 0, 0
    while i < len(ids):
        if ids[i] != image_token_id:
            for c in range(3):
                out[c].append(nxt)
            nxt += 1
            i += 1
            continue
        if img >= len(grids):
            raise ValueError("more image runs in the prompt than grids")
        t, h, w = grids[img]
        h, w = h // spatial_merge, w // spatial_merge
        n = t * h * w
        if ids[i:i + n] != [image_token_id] * n:
            raise ValueError(f"image {img} needs a run of {n} image tokens")
        for tt in range(t):
            for hh in range(h):
                for ww in range(w):
                    out[0].append(nxt + tt)
                    out[1].append(nxt + hh)
                    out[2].append(nxt + ww)
        nxt += max(t, h, w)
        i += n
        img += 1
    return torch.tensor(out, dtype=torch.int32), nxt - len(ids)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on ``x [T, H, D]`` for the first ``rotary_dim`` features (fp32 math)."""
    rd = cos_sin.shape[-1]
    half = rd // 2
    cs = cos_sin[positions.long()]
    cos, sin = cs[:, None, :half].float(), cs[:, None, half:].float()
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:rd]
    out = xf.clone()
    out[..., :half] = x1 * cos - x2 * sin
    out[..., half:rd] = x2 * cos + x1 * sin
    return out.to(x.dtype)


def _head_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y.to(x.dtype).float() * w.float()).to(x.dtype)


def rope_kv_write(qkv: torch.Tensor, kv_layer: torch.Tensor, meta: StepMeta, cos_sin: torch.Tensor,
                  num_q_heads: int, num_kv_heads: int, head_dim: int,
                  q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None,
                  eps: float = 1e-6) -> torch.Tensor:
    """Split packed ``qkv [T,(Hq+2Hkv)D]``, optional per-head q/k RMSNorm, RoPE on q and k,
    write k and v into the paged cache ``kv_layer [pages, 2, Hkv, P, D]``; returns ``q [T,Hq,D]``.
    """
    t = qkv.shape[0]
    q, k, v = qkv.split([num_q_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * head_dim], dim=-1)
    q = q.reshape(t, num_q_heads, head_dim)
    k = k.reshape(t, num_kv_heads, head_dim)
    v = v.reshape(t, num_kv_heads, head_dim)
    if q_norm_w is not None:
        q = _head_rmsnorm(q, q_norm_w, eps)
    if k_norm_w is not None:
        k = _head_rmsnorm(k, k_norm_w, eps)
    pos = meta.positions
    if meta.rope_rows is not None:          # multimodal RoPE: per-row tables prepared by the model
        cos_sin, pos = meta.rope_rows, meta.rope_pos
    q = apply_rope(q, pos, cos_sin)
    k = apply_rope(k, pos, cos_sin)
    p = meta.page_size
    sid = meta.seq_ids.long()
    if meta.kv_offsets is not None:
        slot = meta.past_len.long()[sid] + meta.kv_offsets.long()
    else:
        slot = meta.past_len.long()[sid] + (torch.arange(t, device=qkv.device) - meta.q_start.long()[sid])
    page = meta.page_table.long()[sid, slot // p]
    kv_layer[page, 0, :, slot % p, :] = k.to(kv_layer.dtype)
    kv_layer[page, 1, :, slot % p, :] = v.to(kv_layer.dtype)
    return q


def rope_q(q: torch.Tensor, meta: StepMeta, cos_sin: torch.Tensor, num_q_heads: int, head_dim: int,
           q_norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6) -> torch.Tensor:
    """Query side of :func:`rope_kv_write` alone (KV-shared layers attend over another layer's cache and write nothing):
    ``q [T, Hq·D]`` → optional per-head RMSNorm, RoPE → ``[T, Hq, D]``."""
    t = q.shape[0]
    q = q.reshape(t, num_q_heads, head_dim)
    if q_norm_w is not None:
        q = _head_rmsnorm(q, q_norm_w, eps)
    pos = meta.positions
    if meta.rope_rows is not None:
        cos_sin, pos = meta.rope_rows, meta.rope_pos
    return apply_rope(q, pos, cos_sin)


def gather_kv(kv_layer: torch.Tensor, page_table_row: torch.Tensor, length: int, page_size: int
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense ``k, v [Hkv, length, D]`` of one sequence from the paged pool."""
    n_pages = (length + page_size - 1) // page_size
    pages = page_table_row[:n_pages].long()
    blk = kv_layer[pages]                      # [n, 2, Hkv, P, D]
    k = blk[:, 0].permute(1, 0, 2, 3).reshape(blk.shape[2], -1, blk.shape[-1])[:, :length]
    v = blk[:, 1].permute(1, 0, 2, 3).reshape(blk.shape[2], -1, blk.shape[-1])[:, :length]
    return k, v


def paged_attention(q: torch.Tensor, kv_layer: torch.Tensor, meta: StepMeta, scale: float,
                    sliding_window: Optional[int] = None, sinks: Optional[torch.Tensor] = None, causal: bool = True) -> torch.Tensor:
    """Causal GQA attention of the step's rows over the paged cache (which already holds this
    step's keys/values).  Row ``i`` of a sequence sees cache slots ``[0, past + i]``
    (bottom-right aligned causal mask), optionally limited to a sliding window, or the tree
    mask for speculative verification.  ``q [T,Hq,D]`` → ``[T,Hq,D]``."""
    t, hq, d = q.shape
    hkv = kv_layer.shape[2]
    g = hq // hkv
    out = torch.empty_like(q)
    for s in range(meta.num_seqs):
        r0, ql, past = int(meta.q_start[s]), int(meta.q_len[s]), int(meta.past_len[s])
        if ql == 0:
            continue
        total = past + ql
        k, v = gather_kv(kv_layer, meta.page_table[s], total, meta.page_size)
        qs = q[r0:r0 + ql].float().permute(1, 0, 2)                      # [Hq, ql, D]
        kf = k.float().repeat_interleave(g, dim=0)                        # [Hq, total, D]
        vf = v.float().repeat_interleave(g, dim=0)
        sc = torch.matmul(qs, kf.transpose(1, 2)) * scale                 # [Hq, ql, total]
        rows = torch.arange(ql, device=q.device)[:, None]
        cols = torch.arange(total, device=q.device)[None, :]
        if meta.tree_mask is not None:
            words = meta.tree_mask[r0:r0 + ql].long()                     # [ql, W]
            new_c = (cols - past).clamp(min=0)
            bit = (words.gather(1, (new_c // 32).expand(ql, -1)) >> (new_c % 32)) & 1
            allowed = (cols < past) | ((cols >= past) & (bit == 1))
        elif not causal:
            allowed = (cols < total) & (rows >= 0)
        else:
            allowed = cols <= past + rows
        if sliding_window is not None and causal:
            allowed = allowed & (cols > past + rows - sliding_window)
        sc = sc.masked_fill(~allowed[None], float("-inf"))
        if sinks is not None:
            sink = sinks.float().view(hq, 1, 1).expand(hq, ql, 1)
            pr = torch.softmax(torch.cat([sc, sink], dim=-1), dim=-1)[..., :-1]
        else:
            pr = torch.softmax(sc, dim=-1)
        out[r0:r0 + ql] = torch.matmul(pr, vf).permute(1, 0, 2).to(q.dtype)
    return out


# ------------------------------------------------------------------------------------------
# NVFP4 (E2M1 values, E4M3 scale per 16 elements, fp32 global scale)

E2M1_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
FP4_MAX = 6.0
E4M3_MAX = 448.0


def _e2m1_table(device) -> torch.Tensor:
    lv = torch.tensor(E2M1_LEVELS, dtype=torch.float32, device=device)
    return torch.cat([lv, -lv])


def fp4_encode(x: torch.Tensor) -> torch.Tensor:
    """Round fp32 values (already divided by their scale) to E2M1 codes 0..15, ties to even."""
    ax = x.abs().clamp(max=FP4_MAX)
    # thresholds between consecutive levels; ties go to the code with an even mantissa bit
    code = torch.zeros_like(ax, dtype=torch.uint8)
    bounds = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
    tie_up = (False, True, False, True, False, True, False)   # at a tie, go up iff the upper code is even
    for i, (b, up) in enumerate(zip(bounds, tie_up)):
        code = torch.where((ax > b) | ((ax == b) & up), torch.full_like(code, i + 1), code)
    sign = (x < 0) | ((x == 0) & (torch.signbit(x)))
    return code | (sign.to(torch.uint8) << 3)


def fp4_pack(codes: torch.Tensor) -> torch.Tensor:
    """Pack ``[..., K]`` codes into ``[..., K/2]`` bytes, even index in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def fp4_unpack(packed: torch.Tensor) -> torch.Tensor:
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def nvfp4_quantize(x: torch.Tensor, global_scale: Optional[torch.Tensor] = None
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Quantise ``x [..., K]`` to NVFP4.

    Returns ``(packed uint8 [..., K/2], block_scale float8_e4m3fn [..., K/16], global_scale fp32)``
    with ``x ≈ e2m1 * block_scale * global_scale`` and ``global_scale = amax / (6 * 448)``."""
    xf = x.float()
    if global_scale is None:
        global_scale = (xf.abs().amax() / (FP4_MAX * E4M3_MAX)).clamp(min=1e-12)
    gs = global_scale.float().reshape(())
    blocks = xf.reshape(*xf.shape[:-1], xf.shape[-1] // 16, 16)
    amax = blocks.abs().amax(-1)
    sf = (amax / FP4_MAX / gs).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
    sff = sf.float() * gs
    scaled = torch.where(sff[..., None] > 0, blocks / sff[..., None].clamp(min=1e-30), torch.zeros_like(blocks))
    codes = fp4_encode(scaled).reshape(xf.shape)
    return fp4_pack(codes), sf, gs


def nvfp4_dequantize(packed: torch.Tensor, block_scale: torch.Tensor, global_scale: torch.Tensor,
                     dtype=torch.float32) -> torch.Tensor:
    codes = fp4_unpack(packed).long()
    vals = _e2m1_table(packed.device)[codes]
    k = vals.shape[-1]
    vals = vals.reshape(*vals.shape[:-1], k // 16, 16) * block_scale.float()[..., None]
    return (vals.reshape(*vals.shape[:-2], k) * global_scale.float()).to(dtype)


def nvfp4_act_qdq(x: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    """Fake-quantise activations exactly as the W4A4 GEMM sees them."""
    p, sf, gs = nvfp4_quantize(x, global_scale)
    return nvfp4_dequantize(p, sf, gs, x.dtype)


def nvfp4_linear(x: torch.Tensor, w_packed: torch.Tensor, w_scale: torch.Tensor, w_scale_2: torch.Tensor,
                 input_scale: Optional[torch.Tensor], bias: Optional[torch.Tensor] = None,
                 quantize_activations: bool = True) -> torch.Tensor:
    w = nvfp4_dequantize(w_packed, w_scale, w_scale_2)
    xa = x.float()
    if quantize_activations:
        gs = input_scale if input_scale is not None else None
        p, sf, g = nvfp4_quantize(xa, gs)
        xa = nvfp4_dequantize(p, sf, g)
    y = xa @ w.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def int4_awq_dequantize(qweight: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor], group: int
                        ) -> torch.Tensor:
    """ModelOpt-prepacked INT4: ``qweight [out/2, in]`` uint8 (row 2r in the low nibble, 2r+1 high),
    ``scales [out, in/group]``; symmetric when ``zeros`` is None (offset 8)."""
    lo, hi = (qweight & 0xF).float(), (qweight >> 4).float()
    w = torch.stack([lo, hi], dim=1).reshape(qweight.shape[0] * 2, qweight.shape[1])
    z = 8.0 if zeros is None else zeros.float().repeat_interleave(group, dim=1)
    return (w - z) * scales.float().repeat_interleave(group, dim=1)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


# ------------------------------------------------------------------------------------------
# MoE


def moe_route_softmax_topk(logits: torch.Tensor, top_k: int, renormalize: bool = True
                           ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax over experts then top-k by value (ties → lower index); weights fp32 ``[T,k]``."""
    probs = torch.softmax(logits.float(), dim=-1)
    # torch.topk is not guaranteed stable on ties; sort descending with a stable sort instead
    order = torch.sort(probs, dim=-1, descending=True, stable=True)
    w, idx = order.values[..., :top_k], order.indices[..., :top_k]
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, idx.to(torch.int32)


def moe_route_sigmoid_group_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, n_group: int,
                                 topk_group: int, renormalize: bool, scaling: float
                                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    s = torch.sigmoid(logits.float())
    sel = s + (bias.float() if bias is not None else 0.0)
    t, e = sel.shape
    grp = sel.view(t, n_group, e // n_group)
    gscore = grp.topk(min(2, e // n_group), dim=-1).values.sum(-1)
    gidx = gscore.topk(topk_group, dim=-1).indices
    gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1.0)
    masked = sel.masked_fill(gmask.repeat_interleave(e // n_group, dim=1) == 0, float("-inf"))
    idx = torch.sort(masked, dim=-1, descending=True, stable=True).indices[..., :top_k]
    w = s.gather(1, idx)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scaling, idx.to(torch.int32)


def moe_ffn(x: torch.Tensor, topk_w: torch.Tensor, topk_idx: torch.Tensor, w13, w2, act: str = "swiglu"
            ) -> torch.Tensor:
    """``y = Σ_k w_k · down_e(act(gate_up_e x))`` with expert weight callables or dense tensors.

    ``w13 [E, 2I, H]`` (gate rows first, then up; ``[E, I, H]`` when ``act == 'relu2'``), ``w2 [E, H, I]``."""
    t, h = x.shape
    out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
    for e in topk_idx.unique().tolist():
        rows, slot = (topk_idx == e).nonzero(as_tuple=True)
        if rows.numel() == 0:
            continue
        xe = x[rows].float()
        hmid = xe @ w13[e].float().t()
        if act == "swiglu":
            g, u = hmid.chunk(2, dim=-1)
            hmid = F.silu(g) * u
        else:
            hmid = F.relu(hmid).pow(2)
        hmid = hmid.to(x.dtype).float()
        ye = hmid @ w2[e].float().t()
        out.index_add_(0, rows, ye * topk_w[rows, slot].float()[:, None])
    return out.to(x.dtype)


# ------------------------------------------------------------------------------------------
# Mamba2 / conv1d / gated delta rule


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], conv_state: torch.Tensor,
                  meta: StepMeta, activation: bool = True) -> torch.Tensor:
    """Depthwise causal conv over packed rows ``x [T,C]`` with per-sequence rolling history
    ``conv_state [rows, C, W-1]`` (oldest first) addressed by ``meta.slot_ids``; state updated in place.
    A sequence with ``past_len == 0`` starts from zero history."""
    t, c = x.shape
    w = weight.shape[-1]
    wf = weight.reshape(c, w).float()
    out = torch.empty_like(x)
    for s in range(meta.num_seqs):
        r0, ql, past, slot = int(meta.q_start[s]), int(meta.q_len[s]), int(meta.past_len[s]), int(meta.slot_ids[s])
        if ql == 0:
            continue
        hist = conv_state[slot].float() if past > 0 else torch.zeros(c, w - 1, device=x.device)
        seq = torch.cat([hist, x[r0:r0 + ql].float().t()], dim=1)            # [C, W-1+ql]
        y = F.conv1d(seq[None], wf[:, None, :], None if bias is None else bias.float(), groups=c)[0]
        if activation:
            y = F.silu(y)
        out[r0:r0 + ql] = y.t().to(x.dtype)
        conv_state[slot] = seq[:, -(w - 1):].to(conv_state.dtype)
    return out


def ssm_scan(x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, D: torch.Tensor,
             dt_bias: torch.Tensor, ssm_state: torch.Tensor, meta: StepMeta, z: Optional[torch.Tensor] = None,
             dt_softplus: bool = True, dt_limit: float = 0.0) -> torch.Tensor:
    """Mamba2 selective-state recurrence over packed rows (sequential, fp32).

    ``x [T,nh,hd]``, ``dt [T,nh]``, ``A [nh]`` (negative), ``B,C [T,G,N]``, ``D [nh]``,
    ``ssm_state [rows, nh, hd, N]`` fp32 updated in place; returns ``y [T,nh,hd]``."""
    t, nh, hd = x.shape
    g = B.shape[1]
    hpg = nh // g
    out = torch.empty_like(x)
    for s in range(meta.num_seqs):
        r0, ql, past, slot = int(meta.q_start[s]), int(meta.q_len[s]), int(meta.past_len[s]), int(meta.slot_ids[s])
        if ql == 0:
            continue
        h = ssm_state[slot].float() if past > 0 else torch.zeros(nh, hd, B.shape[-1], device=x.device)
        for i in range(r0, r0 + ql):
            d = dt[i].float() + dt_bias.float()
            if dt_softplus:
                d = torch.where(d > 20.0, d, F.softplus(d))
            if dt_limit > 0:
                d = d.clamp(max=dt_limit)
            dA = torch.exp(A.float() * d)                                    # [nh]
            Bh = B[i].float().repeat_interleave(hpg, dim=0)                   # [nh, N]
            Ch = C[i].float().repeat_interleave(hpg, dim=0)
            xi = x[i].float()                                                 # [nh, hd]
            h = h * dA[:, None, None] + (d[:, None] * xi)[:, :, None] * Bh[:, None, :]
            y = (h * Ch[:, None, :]).sum(-1) + D.float()[:, None] * xi
            if z is not None:
                y = y * F.silu(z[i].float())
            out[i] = y.to(x.dtype)
        ssm_state[slot] = h.to(ssm_state.dtype)
    return out


def gated_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, b: torch.Tensor,
                     A_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, meta: StepMeta) -> torch.Tensor:
    """Gated delta rule over packed rows.  ``q,k [T,hk,K]``, ``v [T,hv,V]``, ``a,b [T,hv]``,
    ``state [rows, hv, K, V]`` fp32 updated in place; returns ``o [T,hv,V]``."""
    t, hk, kd = q.shape
    hv = v.shape[1]
    rep = hv // hk
    out = torch.empty_like(v)
    for s in range(meta.num_seqs):
        r0, ql, past, slot = int(meta.q_start[s]), int(meta.q_len[s]), int(meta.past_len[s]), int(meta.slot_ids[s])
        if ql == 0:
            continue
        H = state[slot].float() if past > 0 else torch.zeros(hv, kd, v.shape[-1], device=q.device)
        for i in range(r0, r0 + ql):
            qi = q[i].float()
            ki = k[i].float()
            qi = qi * torch.rsqrt(qi.pow(2).sum(-1, keepdim=True) + 1e-6) * (kd ** -0.5)
            ki = ki * torch.rsqrt(ki.pow(2).sum(-1, keepdim=True) + 1e-6)
            qi = qi.repeat_interleave(rep, dim=0)
            ki = ki.repeat_interleave(rep, dim=0)                              # [hv, K]
            gdec = torch.exp(-torch.exp(A_log.float()) * F.softplus(a[i].float() + dt_bias.float()))
            beta = torch.sigmoid(b[i].float())
            H = H * gdec[:, None, None]
            pred = torch.einsum("hkv,hk->hv", H, ki)
            delta = beta[:, None] * (v[i].float() - pred)
            H = H + ki[:, :, None] * delta[:, None, :]
            out[i] = torch.einsum("hkv,hk->hv", H, qi).to(v.dtype)
        state[slot] = H.to(state.dtype)
    return out


# ------------------------------------------------------------------------------------------
# sampling


def apply_token_bitmask(logits: torch.Tensor, bitmask: torch.Tensor) -> torch.Tensor:
    """Mask (−1e30) every vocabulary entry whose bit is 0 in ``bitmask [rows, ceil(V/32)]`` int32."""
    v = logits.shape[-1]
    idx = torch.arange(v, device=logits.device)
    bits = (bitmask.long()[:, idx // 32] >> (idx % 32)) & 1
    return torch.where(bits == 1, logits, torch.full_like(logits, -1e30))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniforms: torch.Tensor) -> torch.Tensor:
    """Per-row top-k / top-p sampling.  ``temperature < 1e-3`` means greedy.  ``uniforms [rows]`` in
    [0,1) make the draw independent of batch composition (``cpp/sampler/sampling.h:56-160``)."""
    rows, v = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    for r in range(rows):
        temp = float(temperature[r])
        if temp < 1e-3:
            out[r] = int(torch.argmax(logits[r].float()))
            continue
        lg = logits[r].float() / temp
        k = int(top_k[r])
        p = float(top_p[r])
        srt = torch.sort(lg, descending=True, stable=True)
        vals, idx = srt.values, srt.indices
        if k > 0:
            vals, idx = vals[:k], idx[:k]
        probs = torch.softmax(vals, dim=-1)
        if p < 1.0:
            cum = probs.cumsum(-1)
            keep = (cum - probs) < p
            probs = torch.where(keep, probs, torch.zeros_like(probs))
            probs = probs / probs.sum()
        cum = probs.cumsum(-1)
        j = int(torch.searchsorted(cum, torch.tensor(float(uniforms[r]) * float(cum[-1]), device=cum.device)).clamp(max=probs.numel() - 1))
        out[r] = int(idx[j])
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    return torch.argmax(logits.float(), dim=-1).to(torch.int32)


# ------------------------------------------------------------------------------------------
# speculative decoding


def spec_accept_greedy(target_tokens: torch.Tensor, tree_tokens: torch.Tensor, parents: torch.Tensor, max_path: int,
                       force_len: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Greedy tree acceptance.  Node 0 is the root; parents precede children.  From the root, follow
    the lowest-index child whose token equals the target arg-max at the current node.  Returns
    ``(path [B, max_path] node indices, path_len [B] (root included), bonus [B])`` where the bonus
    token is the target arg-max at the last accepted node.  ``force_len > 0`` (an int or a per-sequence tensor) ignores
    tokens and follows first children until the path holds that many nodes (benchmark mode,
    ``cpp/kernels/speculative/forceAcceptanceKernels.cu``)."""
    b, n = tree_tokens.shape
    path = torch.zeros(b, max_path, dtype=torch.int32, device=tree_tokens.device)
    plen = torch.ones(b, dtype=torch.int32, device=tree_tokens.device)
    bonus = torch.zeros(b, dtype=torch.int32, device=tree_tokens.device)
    for i in range(b):
        cur, ln = 0, 1
        fl = int(force_len[i]) if isinstance(force_len, torch.Tensor) else int(force_len)
        while ln < max_path and not (fl > 0 and ln >= fl):
            want = int(target_tokens[i, cur])
            nxt = -1
            for c in range(cur + 1, n):
                if int(parents[i, c]) == cur and (fl > 0 or int(tree_tokens[i, c]) == want):
                    nxt = c
                    break
            if nxt < 0:
                break
            cur = nxt
            path[i, ln] = cur
            ln += 1
        plen[i] = ln
        bonus[i] = target_tokens[i, cur]
    return path, plen, bonus


def sampling_probs(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """The distribution the sampler draws from: softmax(logits / T) restricted to the top-k tokens and the smallest
    top-p nucleus, renormalised (fp32, ``[rows, V]``)."""
    x = logits.float() / max(float(temperature), 1e-6)
    if top_k and top_k < x.shape[-1]:
        kth = x.topk(top_k, dim=-1).values[..., -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    p = torch.softmax(x, dim=-1)
    if top_p < 1.0:
        sp, si = p.sort(dim=-1, descending=True)
        keep = (sp.cumsum(-1) - sp) < top_p                   # a token stays while the mass before it is below top_p
        sp = sp * keep
        p = torch.zeros_like(p).scatter_(-1, si, sp)
        p = p / p.sum(-1, keepdim=True)
    return p


def token_logprobs(logits: torch.Tensor, tokens: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Log-probability of ``tokens[row]`` and the ``k`` most likely tokens (ordered by probability, ties → the lower id) of every
    row under ``softmax(logits[row])``: ``(chosen [rows], top_ids [rows, k] int32, top_values [rows, k])`` fp32."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    chosen = lp.gather(1, tokens.long().to(lp.device)[:, None])[:, 0]
    if k <= 0:
        return chosen, torch.empty(lp.shape[0], 0, dtype=torch.int32, device=lp.device), torch.empty(lp.shape[0], 0, device=lp.device)
    order = lp.sort(dim=-1, descending=True, stable=True)
    return chosen, order.indices[:, :k].to(torch.int32), order.values[:, :k]


def spec_accept_sampling(target_probs: torch.Tensor, tree_tokens: torch.Tensor, parents: torch.Tensor, max_path: int,
                         uniforms: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Lossless tree acceptance for sampled requests (``cpp/kernels/speculative/speculativeSamplingKernels.cu`` in the
    reference).  The draft's children of a node are fixed candidates, i.e. point-mass proposals: candidate ``c`` is
    accepted with probability ``p(c)`` under the node's current target distribution ``p``; on rejection ``c`` is removed
    from ``p`` and ``p`` renormalised (the residual distribution), and the next sibling is tried.  When no child is
    accepted — or the node is a leaf — the bonus token is drawn from what is left of ``p``.  Every emitted token is then
    distributed exactly as if it had been sampled from the target alone.

    ``target_probs [B, N, V]`` (see :func:`sampling_probs`), ``uniforms [B, max_path, K+1]`` in [0, 1): one per sibling
    trial and one for the bonus draw at each depth.  Returns ``(path, path_len, bonus)`` like the greedy form."""
    b, n = tree_tokens.shape
    dev = tree_tokens.device
    path = torch.zeros(b, max_path, dtype=torch.int32, device=dev)
    plen = torch.ones(b, dtype=torch.int32, device=dev)
    bonus = torch.zeros(b, dtype=torch.int32, device=dev)
    par = parents.tolist()
    tok = tree_tokens.tolist()
    u = uniforms.tolist()
    for i in range(b):
        cur, ln = 0, 1
        while True:
            p = target_probs[i, cur].double().clone()
            depth = ln - 1
            nxt = -1
            if ln < max_path:
                trial = 0
                for c in range(cur + 1, n):
                    if par[i][c] != cur:
                        continue
                    mass = float(p.sum())
                    pc = float(p[tok[i][c]]) / mass if mass > 0 else 0.0
                    if u[i][depth][min(trial, len(u[i][depth]) - 2)] < pc:
                        nxt = c
                        break
                    p[tok[i][c]] = 0.0                          # rejected: the residual excludes this candidate
                    trial += 1
            if nxt < 0:
                mass = float(p.sum())
                if mass <= 0:                                   # every token with mass was a rejected candidate (numerically)
                    p = target_probs[i, cur].double()
                    mass = float(p.sum())
                cdf = (p / mass).cumsum(0)
                bonus[i] = int(torch.searchsorted(cdf, torch.tensor(u[i][depth][-1], dtype=torch.float64)).clamp(max=p.numel() - 1))
                break
            cur = nxt
            path[i, ln] = cur
            ln += 1
        plen[i] = ln
    return path, plen, bonus


def kv_commit_path(pool: torch.Tensor, page_table: torch.Tensor, past_len: torch.Tensor, path: torch.Tensor,
                   path_len: torch.Tensor) -> None:
    """Compact the accepted path in the paged cache ``pool [L, pages, 2, Hkv, P, D]``: the entry at
    slot ``past + path[j]`` moves to slot ``past + j`` (``j ≥ 1``), in place."""
    p = pool.shape[4]
    for i in range(path.shape[0]):
        past, m = int(past_len[i]), int(path_len[i])
        rows = []
        for j in range(1, m):
            s = past + int(path[i, j])
            rows.append(pool[:, int(page_table[i, s // p]), :, :, s % p, :].clone())
        for j, r in zip(range(1, m), rows):
            s = past + j
            pool[:, int(page_table[i, s // p]), :, :, s % p, :] = r


# ------------------------------------------------------------------------------------------
# EAGLE tree construction (host formulation of the device kernels)


def eagle_ancestors(parents: torch.Tensor) -> torch.Tensor:
    """``[B, R, R]`` bool: row r may attend row c iff c is r or one of its ancestors."""
    b, r = parents.shape
    a = torch.eye(r, dtype=torch.bool, device=parents.device).expand(b, r, r).clone()
    p = parents.long().clamp(min=0)
    has = (parents >= 0)[..., None]
    for _ in range(r):
        up = a.gather(1, p[..., None].expand(b, r, r)) & has
        new = a | up
        if torch.equal(new, a):
            break
        a = new
    return a


def eagle_pack_mask(anc: torch.Tensor) -> torch.Tensor:
    """Pack ``[B, R, R]`` bool into int32 words ``[B * R, ceil(R / 32)]`` (bit c of row r)."""
    b, r, _ = anc.shape
    words = (r + 31) // 32
    pad = torch.zeros(b, r, words * 32, dtype=torch.int64, device=anc.device)
    pad[..., :r] = anc.long()
    w = (pad.view(b, r, words, 32) << torch.arange(32, device=anc.device)).sum(-1)
    w = torch.where(w >= 2 ** 31, w - 2 ** 32, w)
    return w.to(torch.int32).view(b * r, words)


def eagle_tree_meta(parents: torch.Tensor, base_pos: torch.Tensor, depth_base: int, pos_offset: int):
    anc = eagle_ancestors(parents)
    depth = (anc.sum(-1) - 1 + depth_base).to(torch.int32)
    pos = (base_pos.to(parents.device).long()[:, None] + depth.long() + pos_offset).to(torch.int32).reshape(-1)
    return eagle_pack_mask(anc), depth, pos


def dflash2_grouped_dynamic_conv(hidden: torch.Tensor, delta: torch.Tensor, base: torch.Tensor, residual: Optional[torch.Tensor],
                                 block: int, group_size: int) -> torch.Tensor:
    """One side of DFlash 2's per-token dynamic grouped depthwise convolution along a proposal block.

    ``hidden [T, H]`` holds whole blocks of ``block`` rows; row ``t`` sits at position ``t % block``.  With ``K`` taps,
    ``out[t, c] = Σ_{k < K, k <= pos(t)} (base[k, c] + delta[t, k, c // group_size]) · hidden[t - k, c]``: a causal filter that never
    reads across a block boundary, whose taps are a fixed per-channel kernel plus a per-token, per-group offset
    (``delta [T, K, H / group_size]``).  With ``residual`` the sum is added to it.  fp32 arithmetic, result in ``hidden``'s type.
    (``cpp/kernels/speculative/dflash2GroupedDynamicConv.cu:80-125``.)"""
    t, h = hidden.shape
    k = base.shape[0]
    x = hidden.float().view(t // block, block, h)
    d = delta.float().view(t // block, block, k, h // group_size).repeat_interleave(group_size, dim=-1)      # [N, B, K, H]
    w = base.float()[None, None] + d
    out = torch.zeros_like(x)
    for tap in range(min(k, block)):
        out[:, tap:] += w[:, tap:, tap] * x[:, :block - tap]
    out = out.view(t, h)
    if residual is not None:
        out = out + residual.float()
    return out.to(hidden.dtype)


def dflash2_selector_walk(cand_ids: torch.Tensor, unary: torch.Tensor, projected: torch.Tensor, anchor: torch.Tensor,
                          pred_codebook: torch.Tensor, succ_codebook: torch.Tensor, temperatures: Optional[torch.Tensor] = None,
                          uniforms: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """DFlash 2's chain selector: walk the proposal slots left to right, scoring slot ``s``'s candidates given the token chosen
    for slot ``s - 1`` (the anchor — the last accepted token — for slot 0):

        score[c] = unary[s, c] + Σ_r P[prev, r] · z[s, r] · Q[cand[s, c], r]

    Greedy rows (no temperature, or one below 1e-3) take the best score (ties → the smaller token id); sampled rows draw from
    ``softmax(score / temperature)`` with ``uniforms[b, s]``.  An id outside the vocabulary contributes no bilinear term.
    Returns ``(tokens [B, S] int64, probabilities [B, S, K] fp32)`` — one-hot on greedy rows.
    (``cpp/kernels/speculative/dflash2CandidateSelector.cu:69-176``.)"""
    b, s, k = cand_ids.shape
    vocab = pred_codebook.shape[0]
    cand = cand_ids.long()
    prev = anchor.long().clone()
    tokens = torch.empty(b, s, dtype=torch.int64, device=cand.device)
    probs = torch.zeros(b, s, k, dtype=torch.float32, device=cand.device)
    pf, qf, z = pred_codebook.float(), succ_codebook.float(), projected.float()
    greedy = torch.ones(b, dtype=torch.bool, device=cand.device) if temperatures is None else temperatures.float() < 1e-3
    for step in range(s):
        ok_prev = (prev >= 0) & (prev < vocab)
        query = pf[prev.clamp(0, vocab - 1)] * z[:, step] * ok_prev[:, None]                        # [B, R]
        c = cand[:, step]
        ok_c = (c >= 0) & (c < vocab)
        dot = torch.einsum("bkr,br->bk", qf[c.clamp(0, vocab - 1)], query) * ok_c
        score = unary[:, step].float() + dot
        # greedy: best score, the smaller token id among equals
        best = score.amax(dim=-1, keepdim=True)
        tie_ids = torch.where(score == best, c, torch.full_like(c, torch.iinfo(torch.int64).max))
        sel = tie_ids.argmin(dim=-1)
        p = torch.nn.functional.one_hot(sel, k).float()
        if not bool(greedy.all()):
            t = temperatures.float().clamp_min(1e-3)
            ps = torch.softmax(score / t[:, None], dim=-1)
            u = uniforms[:, step].float().clamp(0.0, 0.99999994)
            ssel = (ps.cumsum(-1) > u[:, None]).float().argmax(dim=-1)
            ssel = torch.where((ps.cumsum(-1) > u[:, None]).any(-1), ssel, torch.full_like(ssel, k - 1))
            sel = torch.where(greedy, sel, ssel)
            p = torch.where(greedy[:, None], p, ps)
        prev = c.gather(1, sel[:, None])[:, 0]
        tokens[:, step] = prev
        probs[:, step] = p
    return tokens, probs


def markov_chain_propose(logits: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, first_prev: torch.Tensor,
                         temperatures: Optional[torch.Tensor] = None, uniforms: Optional[torch.Tensor] = None) -> torch.Tensor:
    """DSpark's Markov head: proposal step ``i`` picks from ``logits[:, i] + W2 · W1[prev]`` (a rank-``R`` bigram correction of
    the backbone's logits) where ``prev`` is the token chosen at step ``i - 1`` (``first_prev`` — the last accepted token — at
    step 0).  Greedy rows take the arg-max (ties → the lowest id); sampled rows draw from the softmax at their temperature
    with ``uniforms[b, i]``.  ``logits [B, P, V]`` fp32, ``w1 [V, R]``, ``w2 [V, R]`` → tokens ``[B, P]`` int64.
    (``cpp/kernels/speculative/dsparkKernels.cu:746-790`` and the fused greedy step after it.)"""
    b, p, v = logits.shape
    prev = first_prev.long().clamp(0, w1.shape[0] - 1)
    out = torch.empty(b, p, dtype=torch.int64, device=logits.device)
    w1f, w2f = w1.float(), w2.float()
    greedy = torch.ones(b, dtype=torch.bool, device=logits.device) if temperatures is None else temperatures.float() < 1e-3
    for step in range(p):
        corrected = logits[:, step].float() + w1f[prev] @ w2f.t()
        tok = corrected.argmax(dim=-1)
        if not bool(greedy.all()):
            ps = torch.softmax(corrected / temperatures.float().clamp_min(1e-3)[:, None], dim=-1)
            hit = ps.cumsum(-1) > uniforms[:, step].float().clamp(0.0, 0.99999994)[:, None]
            stok = torch.where(hit.any(-1), hit.float().argmax(dim=-1), torch.full_like(tok, v - 1))
            tok = torch.where(greedy, tok, stok)
        out[:, step] = tok
        prev = tok
    return out


def markov_confidence(hidden: torch.Tensor, w1: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, first_prev: torch.Tensor,
                      tokens: torch.Tensor, with_markov: bool) -> torch.Tensor:
    """Per-step acceptance confidence of a DSpark proposal: ``sigmoid(w_h · hidden[b, i] (+ w_m · W1[prev_i]) + bias)`` with
    ``prev_0 = first_prev`` and ``prev_i = tokens[b, i - 1]``; ``weight`` is ``[H]`` or ``[H + R]``.  fp32 ``[B, P]``."""
    h = hidden.shape[-1]
    logit = hidden.float() @ weight.float()[:h] + bias.float().reshape(-1)[0]
    if with_markov:
        prev = torch.cat([first_prev.long()[:, None], tokens.long()[:, :-1]], dim=1).clamp(0, w1.shape[0] - 1)
        logit = logit + w1.float()[prev] @ weight.float()[h:]
    return torch.sigmoid(logit)


_SPS_DRAFT, _SPS_VERIFY_BASE, _SPS_VERIFY_TOKEN, _SPS_ACCEPT = 0.50, 1.00, 0.45, 0.02


def confidence_proposal_lengths(conf: torch.Tensor, mode: str, value: float, min_len: int = 1, max_len: int = 0) -> torch.Tensor:
    """Proposal length per sequence from per-step confidences ``[B, P]`` (the survival probability of step ``i`` is the product
    of the confidences up to ``i``).

    ``"threshold"``: the longest prefix whose survival stays at or above ``value`` (``value <= 0``: the maximum length).
    ``"sps"``: the length that maximises expected emitted tokens per unit cost, ``(1 + Σ survival) / (0.5 + 1.0 + 0.45 · (len + 1)
    + 0.02 · len)``, stopping once survival falls below the floor ``value``.
    Lengths are clamped to ``[min_len, max_len]`` (``max_len <= 0``: P).  (``dsparkKernels.cu:664-744``.)"""
    b, p = conf.shape
    lo = max(1, min(p, min_len))
    hi = max(lo, min(p, p if max_len <= 0 else max_len))
    out = torch.empty(b, dtype=torch.int64)
    c = conf.float().cpu()
    for i in range(b):
        if mode == "threshold":
            if value <= 0:
                out[i] = hi
                continue
            surv, sel = 1.0, lo
            for step in range(hi):
                surv *= float(c[i, step])
                if surv >= value:
                    sel = step + 1
                else:
                    break
        elif mode == "sps":
            floor = min(1.0, max(0.0, value))
            surv, expected, best, sel = 1.0, 1.0, -float("inf"), lo
            for step in range(hi):
                length = step + 1
                surv *= float(c[i, step])
                expected += surv
                if length >= lo:
                    score = expected / max(_SPS_DRAFT + _SPS_VERIFY_BASE + _SPS_VERIFY_TOKEN * (length + 1) + _SPS_ACCEPT * length, 1e-6)
                    if score > best:
                        best, sel = score, length
                if floor > 0 and surv < floor and length >= lo:
                    break
        else:
            raise ValueError(f"unknown proposal-length schedule {mode!r}")
        out[i] = max(lo, min(hi, sel))
    return out


def lattice_chain_walk(cand_ids: torch.Tensor, transition: torch.Tensor, temperatures: Optional[torch.Tensor] = None,
                       uniforms: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Walk a candidate lattice slot by slot: ``transition[b, s, prev, next]`` scores candidate ``next`` of slot ``s`` given the
    index chosen at slot ``s - 1`` (index 0 before the first slot).  Greedy rows take the best score (ties → the lowest index)
    with a one-hot distribution; sampled rows draw from ``softmax(row / temperature)`` by inverse CDF on ``uniforms[b, s]``.
    Returns ``(tokens [B, S] int64, probabilities [B, S, K] fp32)``.  (``cpp/kernels/speculative/lilicorrChainWalk.h``.)"""
    b, s, k = cand_ids.shape
    dev = cand_ids.device
    prev = torch.zeros(b, dtype=torch.int64, device=dev)
    tokens = torch.empty(b, s, dtype=torch.int64, device=dev)
    probs = torch.zeros(b, s, k, dtype=torch.float32, device=dev)
    greedy = torch.ones(b, dtype=torch.bool, device=dev) if temperatures is None else temperatures.float() < 1e-3
    rows = torch.arange(b, device=dev)
    for step in range(s):
        row = transition[rows, step, prev].float()                                  # [B, K]
        sel = row.argmax(dim=-1)                                                     # first maximum = lowest index
        p = torch.nn.functional.one_hot(sel, k).float()
        if not bool(greedy.all()):
            ps = torch.softmax(row / temperatures.float().clamp_min(1e-3)[:, None], dim=-1)
            hit = ps.cumsum(-1) > uniforms[:, step].float().clamp(0.0, 0.99999994)[:, None]
            ssel = torch.where(hit.any(-1), hit.float().argmax(dim=-1), torch.full_like(sel, k - 1))
            sel = torch.where(greedy, sel, ssel)
            p = torch.where(greedy[:, None], p, ps)
        tokens[:, step] = cand_ids[rows, step, sel]
        probs[:, step] = p
        prev = sel
    return tokens, probs


def candidate_rescore(hidden: torch.Tensor, lm_head: torch.Tensor, cand: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exact scores of a candidate set: ``logit[r, c] = lm_head[cand[r, c]] · hidden[r]`` in fp32, candidates reordered by
    (logit descending, token id ascending; a non-finite logit counts as -inf), log-softmax over the set.  Returns
    ``(ids [R, Kc] int32, log-probabilities [R, Kc] fp32)``."""
    cand = cand.long()
    logits = torch.einsum("rkh,rh->rk", lm_head[cand].float(), hidden.float())
    finite = torch.isfinite(logits)
    ranked = torch.where(finite, logits, torch.full_like(logits, float("-inf")))
    by_id = cand.argsort(dim=-1, stable=True)                              # ascending ids first, then a stable sort by value
    ranked, cand, finite = ranked.gather(-1, by_id), cand.gather(-1, by_id), finite.gather(-1, by_id)
    order = ranked.sort(dim=-1, descending=True, stable=True).indices
    ranked, cand, finite = ranked.gather(-1, order), cand.gather(-1, order), finite.gather(-1, order)
    lse = torch.logsumexp(ranked, dim=-1, keepdim=True)
    lp = torch.where(finite, ranked - lse, torch.full_like(ranked, float("-inf")))
    return cand.to(torch.int32), lp


def low_rank_candidate_head(hidden: torch.Tensor, down_proj: torch.Tensor, up_proj: torch.Tensor, lm_head: torch.Tensor,
                            num_candidates: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Candidate head of EAGLE-4 drafts (``tensorrt_edgellm/models/ops.py:636-679``): the ``num_candidates`` tokens with the
    largest low-rank scores ``A (B h)`` (``B = down_proj [r, H]``, ``A = up_proj [V, r]``; ``B h`` accumulates in fp32 and is
    rounded to the weights' 16-bit type, the scores are fp32; ties go to the smaller id, NaN ranks last), then
    :func:`candidate_rescore` with the exact ``lm_head`` rows."""
    h32 = hidden.float()
    proj = (h32 @ down_proj.float().t()).to(down_proj.dtype if down_proj.dtype != torch.float32 else torch.float16)
    scores = proj.float() @ up_proj.float().t()
    scores = torch.where(torch.isnan(scores), torch.full_like(scores, float("-inf")), scores)
    cand = scores.sort(dim=-1, descending=True, stable=True).indices[:, :num_candidates]
    return candidate_rescore(hidden, lm_head, cand)


def eagle_select_verify(p_sc, p_tok, p_par, p_dep, root, keep: int):
    b, npool = p_sc.shape
    dev = p_sc.device
    order = torch.sort(p_sc.float(), dim=1, descending=True, stable=True).indices[:, :keep]
    sel = torch.sort(order, dim=1).values                                 # pool order = parents first
    inv = torch.zeros((b, npool), dtype=torch.long, device=dev)           # a parent that was not kept re-attaches to the root
    inv.scatter_(1, sel, torch.arange(1, keep + 1, device=dev).expand(b, keep))
    spar = p_par.long().gather(1, sel)
    parents = torch.where(spar < 0, torch.zeros_like(spar), inv.gather(1, spar.clamp(min=0)))
    i32 = torch.int32
    tok = torch.cat([root.to(dev).long()[:, None], p_tok.long().gather(1, sel)], dim=1).to(i32)
    par = torch.cat([torch.full((b, 1), -1, device=dev, dtype=torch.long), parents], dim=1).to(i32)
    dep = torch.cat([torch.zeros(b, 1, dtype=torch.long, device=dev), p_dep.long().gather(1, sel)], dim=1).to(i32)
    return tok, par, dep


# ------------------------------------------------------------------------------------------
# FP8 (E4M3) KV storage: host formulation of csrc/kernels/kv_fp8.cu


def kv_fp8_load(kv_layer: torch.Tensor, stage: torch.Tensor, meta, scales: torch.Tensor, window: int = 0) -> None:
    psz = kv_layer.shape[3]
    table = meta.page_table.cpu()
    sc = scales.float().view(2, 1, 1, 1).to(stage.device)
    for s in range(meta.num_seqs):
        past = int(meta.past_len[s])
        for lp in range((past + psz - 1) // psz):
            page = int(table[s, lp])
            if page >= 0:
                stage[page] = (kv_layer[page].float() * sc).to(stage.dtype)


def kv_fp8_store(kv_layer: torch.Tensor, stage: torch.Tensor, meta, scales: torch.Tensor) -> None:
    psz = kv_layer.shape[3]
    table = meta.page_table.cpu()
    sc = scales.float().view(2, 1, 1).to(stage.device)
    for t in range(meta.num_tokens):
        s = int(meta.seq_ids[t])
        off = int(meta.kv_offsets[t]) if meta.kv_offsets is not None else t - int(meta.q_start[s])
        slot = int(meta.past_len[s]) + off
        page = int(table[s, slot // psz])
        if page < 0:
            continue
        rows = stage[page, :, :, slot % psz].float()                       # [2, Hkv, D]
        q = (rows / sc).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
        kv_layer[page, :, :, slot % psz] = q
        stage[page, :, :, slot % psz] = (q.float() * sc).to(stage.dtype)


# ---- block-draft verification trees ---------------------------------------------------------------------------------

def ddtree_candidates(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-depth candidates of a block draft: the ``k`` most likely tokens of every row of ``logits [B, D, V]`` with their
    log-probabilities over the whole vocabulary.  Returns ``(ids [B, D, k] int32, log-probabilities [B, D, k] fp32)``, each
    list sorted by non-increasing log-probability (ties: lower token id first).
    Parity: ``ddtreeSelectLogitCandidates`` (``cpp/kernels/speculative/ddtreeKernels.h``)."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    # a stable sort on (-log-probability) keeps the lower token id first among equals
    order = torch.argsort(-lp, dim=-1, stable=True)[..., :k]
    return order.to(torch.int32), lp.gather(-1, order)


def ddtree_assemble(cand_ids: torch.Tensor, cand_lp: torch.Tensor, root_tokens: torch.Tensor, num_nodes: int,
                    depth_confidence: Optional[torch.Tensor] = None, survival_threshold: float = 0.0):
    """Best-first assembly of a prefix-closed verification tree from per-depth candidate lists (the positions of a block
    draft are predicted independently of each other, so every node of depth ``d`` has the same candidate children: row
    ``d`` of the table).  Node 0 is the root (score 0).  Each step appends, among the next unused candidate of every node
    already in the tree, the one with the highest prefix score (the sum of log-probabilities along its path, plus
    ``log(confidence)`` of every depth when ``depth_confidence [B, D]`` is given); ties go to the lower parent index, then
    the lower slot, then the lower token id.  A child never outscores its parent, so the result is the ``num_nodes - 1``
    best prefixes of the whole candidate tree.  With a ``survival_threshold`` growth stops below depths whose confidence
    product falls under it.  Returns ``(tokens, parents, depths [B, N] int32, scores [B, N] fp32, valid [B] int32)``;
    rows past ``valid`` are padding (token = root token, parent 0, score -inf).
    Parity: ``ddtreeAssemble`` (``cpp/kernels/speculative/ddtreeKernels.h``)."""
    import heapq
    ids, lps = cand_ids.cpu(), cand_lp.float().cpu()
    b, depth_rows, k = ids.shape
    roots = root_tokens.cpu().tolist()
    conf = depth_confidence.float().cpu() if depth_confidence is not None else None
    tok = torch.zeros(b, num_nodes, dtype=torch.int32)
    par = torch.zeros(b, num_nodes, dtype=torch.int32)
    dep = torch.zeros(b, num_nodes, dtype=torch.int32)
    sc = torch.full((b, num_nodes), float("-inf"))
    valid = torch.zeros(b, dtype=torch.int32)
    for i in range(b):
        tok[i] = int(roots[i])
        sc[i, 0] = 0.0
        gain = [0.0] * depth_rows                 # what entering depth d + 1 adds beside the token's own log-probability
        alive = depth_rows
        if conf is not None:
            prod = 1.0
            for d in range(depth_rows):
                c = min(max(float(conf[i, d]), 0.0), 1.0)
                prod *= c
                gain[d] = math.log(c) if c > 0 else float("-inf")
                if survival_threshold > 0 and prod < survival_threshold and alive == depth_rows:
                    alive = d
        heap: list = []                           # (-score, parent, slot, token)

        def offer(node: int, slot: int) -> None:
            d = int(dep[i, node])
            if d >= alive or slot >= k:
                return
            lp = float(lps[i, d, slot])
            if lp == float("-inf") or gain[d] == float("-inf"):
                return
            heapq.heappush(heap, (-(float(sc[i, node]) + lp + gain[d]), node, slot, int(ids[i, d, slot])))

        offer(0, 0)
        n = 1
        while n < num_nodes and heap:
            neg, node, slot, token = heapq.heappop(heap)
            tok[i, n], par[i, n], dep[i, n], sc[i, n] = token, node, int(dep[i, node]) + 1, -neg
            offer(node, slot + 1)                 # the parent's next candidate
            offer(n, 0)                           # the new node's best child
            n += 1
        valid[i] = n
    dev = cand_ids.device
    return tok.to(dev), par.to(dev), dep.to(dev), sc.to(dev), valid.to(dev)
