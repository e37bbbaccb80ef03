"""Weight-only checkpoint formats ↔ dense ``[out, in]`` matrices.

Every format here is expanded to 16-bit once at load time and then served by the 16-bit tcgen05 GEMM (B200 has
the memory for it; the 4-/8-bit bytes are only a storage and download format).  Layouts follow
``tensorrt_edgellm/models/linear.py:647-920`` (AutoAWQ / GPTQ / ModelOpt INT4), ``tensorrt_edgellm/models/ops.py``
(``fp8_dequantize`` :794, ``mxfp8_*`` :1034, ``q8_0_*`` :1213, ``int8_sq_*`` :1488) and
``tensorrt_edgellm/checkpoint/repacking.py``.  Each decoder has an encoder beside it so the formats can be
produced by the quantisation tool and round-tripped in tests.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)          # 4-bit field i of an AutoAWQ int32 holds logical column 8*c + AWQ_ORDER[i]


def _unpack_int32_nibbles(packed: torch.Tensor, dim: int) -> torch.Tensor:
    """int32 with eight 4-bit fields (field j at bits 4j..4j+3) → uint8, expanding ``dim`` eightfold in field order."""
    p = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(0, 32, 4, dtype=torch.int64)
    if dim == 0:
        out = (p[:, None, :] >> shifts[None, :, None]) & 0xF            # [R, 8, C]
        return out.reshape(-1, packed.shape[1]).to(torch.uint8)
    out = (p[:, :, None] >> shifts[None, None, :]) & 0xF                # [R, C, 8]
    return out.reshape(packed.shape[0], -1).to(torch.uint8)


def _pack_int32_nibbles(vals: torch.Tensor, dim: int) -> torch.Tensor:
    v = vals.to(torch.int64)
    shifts = torch.arange(0, 32, 4, dtype=torch.int64)
    if dim == 0:
        p = (v.reshape(-1, 8, v.shape[1]) << shifts[None, :, None]).sum(1)
    else:
        p = (v.reshape(v.shape[0], -1, 8) << shifts[None, None, :]).sum(2)
    return torch.where(p >= 2 ** 31, p - 2 ** 32, p).to(torch.int32)


# ---- GPTQ: qweight [in/8, out], qzeros [in/g, out/8], scales [in/g, out], g_idx [in] ------------------------------

def decode_gptq(qweight, qzeros, scales, g_idx=None, zero_point_offset: int = 1) -> torch.Tensor:
    q = _unpack_int32_nibbles(qweight, 0).float()                       # [in, out]
    z = _unpack_int32_nibbles(qzeros, 1).float() + zero_point_offset    # [in/g, out]
    n_in = q.shape[0]
    group = n_in // scales.shape[0]
    gi = g_idx.long() if g_idx is not None else torch.arange(n_in) // group
    w = (q - z[gi]) * scales.float()[gi]
    return w.t().contiguous()                                           # [out, in]


def encode_gptq(w: torch.Tensor, group: int = 128, zero_point_offset: int = 1) -> Dict[str, torch.Tensor]:
    wt = w.float().t()                                                  # [in, out]
    n_in, n_out = wt.shape
    wg = wt.reshape(n_in // group, group, n_out)
    lo, hi = wg.amin(1), wg.amax(1)
    scale = ((hi - lo) / 15.0).clamp(min=1e-8)
    zero = torch.round(-lo / scale).clamp(0, 15)
    q = torch.round(wg / scale[:, None] + zero[:, None]).clamp(0, 15)
    return {"qweight": _pack_int32_nibbles(q.reshape(n_in, n_out), 0),
            "qzeros": _pack_int32_nibbles((zero - zero_point_offset) % 16, 1),
            "scales": scale.to(torch.float16), "g_idx": (torch.arange(n_in) // group).to(torch.int32)}


# ---- AutoAWQ: qweight [in, out/8], qzeros [in/g, out/8], scales [in/g, out]; nibble order 0,2,4,6,1,3,5,7 -------------

def _awq_cols(packed: torch.Tensor) -> torch.Tensor:
    u = _unpack_int32_nibbles(packed, 1)                                # field order
    r, c = u.shape
    inv = torch.tensor([AWQ_ORDER.index(j) for j in range(8)])         # logical column j sits in field inv[j]
    return u.reshape(r, c // 8, 8)[:, :, inv].reshape(r, c)


def decode_autoawq(qweight, qzeros, scales) -> torch.Tensor:
    q = _awq_cols(qweight).float()                                      # [in, out]
    z = _awq_cols(qzeros).float()                                       # [in/g, out]
    group = q.shape[0] // scales.shape[0]
    gi = torch.arange(q.shape[0]) // group
    return ((q - z[gi]) * scales.float()[gi]).t().contiguous()


def encode_autoawq(w: torch.Tensor, group: int = 128) -> Dict[str, torch.Tensor]:
    wt = w.float().t()
    n_in, n_out = wt.shape
    wg = wt.reshape(n_in // group, group, n_out)
    lo, hi = wg.amin(1), wg.amax(1)
    scale = ((hi - lo) / 15.0).clamp(min=1e-8)
    zero = torch.round(-lo / scale).clamp(0, 15)
    q = torch.round(wg / scale[:, None] + zero[:, None]).clamp(0, 15).reshape(n_in, n_out)
    order = torch.tensor(AWQ_ORDER)

    def pack(v):
        r, c = v.shape
        return _pack_int32_nibbles(v.reshape(r, c // 8, 8)[:, :, order].reshape(r, c), 1)
    return {"qweight": pack(q), "qzeros": pack(zero), "scales": scale.to(torch.float16)}


# ---- FP8 (E4M3, per-tensor or per-channel scale) ---------------------------------------------------------------------

def decode_fp8(weight, weight_scale=None) -> torch.Tensor:
    w = weight.view(torch.float8_e4m3fn).float()
    if weight_scale is None:
        return w
    s = weight_scale.float()
    return w * (s.reshape(-1, 1) if s.numel() == w.shape[0] else s.reshape(()))


def encode_fp8(w: torch.Tensor, per_channel: bool = False) -> Dict[str, torch.Tensor]:
    wf = w.float()
    amax = wf.abs().amax(1, keepdim=True) if per_channel else wf.abs().amax()
    scale = (amax / 448.0).clamp(min=1e-12)
    return {"weight": (wf / scale).clamp(-448, 448).to(torch.float8_e4m3fn), "weight_scale": scale.reshape(-1) if per_channel else scale.reshape(())}


# ---- INT8 SmoothQuant (per-output-channel weight scale) --------------------------------------------------------------

def decode_int8_sq(weight, weight_scale) -> torch.Tensor:
    return weight.to(torch.int8).float() * weight_scale.float().reshape(-1, 1)


def encode_int8_sq(w: torch.Tensor) -> Dict[str, torch.Tensor]:
    wf = w.float()
    scale = (wf.abs().amax(1) / 127.0).clamp(min=1e-12)
    return {"weight": torch.round(wf / scale[:, None]).clamp(-127, 127).to(torch.int8), "weight_scale": scale}


# ---- MXFP8: E4M3 elements, one E8M0 (power-of-two) scale per 32 ------------------------------------------------------

def decode_mxfp8(weight, weight_scale) -> torch.Tensor:
    w = weight.view(torch.float8_e4m3fn).float()
    e = weight_scale.view(torch.uint8).float()                          # [out, in/32], value 2^(e-127)
    s = torch.exp2(e - 127.0)
    return (w.reshape(w.shape[0], -1, 32) * s[..., None]).reshape(w.shape)


def encode_mxfp8(w: torch.Tensor) -> Dict[str, torch.Tensor]:
    wf = w.float()
    blocks = wf.reshape(wf.shape[0], -1, 32)
    amax = blocks.abs().amax(-1).clamp(min=2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 448.0)).clamp(-127, 127)
    q = (blocks / torch.exp2(e)[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return {"weight": q.reshape(wf.shape), "weight_scale": (e + 127).to(torch.uint8)}


# ---- Q8_0: int8 elements, one fp16 scale per 32 ----------------------------------------------------------------------

def decode_q8_0(weight, weight_scale) -> torch.Tensor:
    w = weight.to(torch.int8).float()
    return (w.reshape(w.shape[0], -1, 32) * weight_scale.float()[..., None]).reshape(w.shape)


def encode_q8_0(w: torch.Tensor) -> Dict[str, torch.Tensor]:
    wf = w.float()
    blocks = wf.reshape(wf.shape[0], -1, 32)
    scale = (blocks.abs().amax(-1) / 127.0).clamp(min=1e-12).to(torch.float16)
    q = torch.round(blocks / scale.float()[..., None]).clamp(-127, 127).to(torch.int8)
    return {"weight": q.reshape(wf.shape), "weight_scale": scale}


def decode_bundle(t: Dict[str, torch.Tensor], quant_type: str, zero_point_offset: int = 1) -> Optional[torch.Tensor]:
    """Dense fp32 ``[out, in]`` of one checkpoint linear stored in a weight-only format; ``None`` if it is plain 16-bit."""
    if "qweight" in t:
        if quant_type == "int4_gptq" or "g_idx" in t:
            return decode_gptq(t["qweight"], t["qzeros"], t["scales"], t.get("g_idx"), zero_point_offset)
        return decode_autoawq(t["qweight"], t["qzeros"], t["scales"])
    w = t.get("weight")
    if w is None:
        return None
    if quant_type == "mxfp8":
        return decode_mxfp8(w, t["weight_scale"])
    if quant_type == "q8_0":
        return decode_q8_0(w, t["weight_scale"])
    if quant_type == "int8_sq" or w.dtype == torch.int8:
        return decode_int8_sq(w, t["weight_scale"])
    if quant_type == "fp8" or w.dtype == torch.float8_e4m3fn:
        return decode_fp8(w, t.get("weight_scale"))
    return None
