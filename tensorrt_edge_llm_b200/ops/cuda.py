"""ctypes binding of the native sm_100a kernel library (``_lib/libtelb_kernels.so``).

Kernels are launched on the current torch CUDA stream with raw device pointers, so they are
captured by ``torch.cuda.graph`` like any other launch.  A missing or stale library is an error:
nothing in this module falls back to PyTorch on a GPU.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict, Optional, Tuple

import torch

from .meta import StepMeta

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_lib", "libtelb_kernels.so")
_lib: Optional[ctypes.CDLL] = None

c_int, c_ll, c_float, c_vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        # fault-injection hook for tests of the failure path (the reference's TRT_EDGELLM_TEST_FAIL_CUTEDSL_MODULE,
        # cpp/kernels/cuteDslModuleLoader.cpp:178): the named library "fails to load" deterministically
        if os.environ.get("TELB_TEST_FAIL_KERNEL_LIBRARY", "") in ("1", os.path.basename(_LIB_PATH)):
            raise RuntimeError(f"native kernel library {_LIB_PATH} failed to load (TELB_TEST_FAIL_KERNEL_LIBRARY is set)")
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f"native kernel library not built: {_LIB_PATH} (run `python -m tensorrt_edge_llm_b200.build`)")
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.telb_last_error.restype = ctypes.c_char_p
    return _lib


LAUNCHES = 0      # kernels of this library launched (or captured) so far in this process


_DEBUG_SYNC = os.environ.get("TELB_DEBUG_SYNC", "0") == "1"     # synchronise after every op so a device error names its op


# Tensors whose pointers were taken for the launch being assembled.  A converted temporary (``x.to(int32)`` written inline
# in an argument list) would otherwise be freed as soon as its pointer is extracted, and the caching allocator may hand the
# same bytes to the next inline conversion of the same call, before the kernel has been enqueued.
_KEEP = threading.local()


def _check(rc: int, what: str, n: int = 1) -> None:
    global LAUNCHES
    held = getattr(_KEEP, "tensors", None)
    if held:
        held.clear()                      # the launch is enqueued: stream order protects the memory from here on
    if rc != 0:
        raise RuntimeError(f"{what} failed: {lib().telb_last_error().decode()}")
    LAUNCHES += n
    if _DEBUG_SYNC and not torch.cuda.is_current_stream_capturing():
        try:
            torch.cuda.synchronize()
        except RuntimeError as e:
            raise RuntimeError(f"device error surfaced after {what}: {e}") from None


def _p(t: Optional[torch.Tensor]):
    if t is None:
        return c_vp(0)
    if not t.is_cuda:        # a host pointer handed to a kernel is a device fault, not an exception
        raise ValueError(f"kernel argument of shape {tuple(t.shape)} lives on {t.device}, not on the GPU")
    held = getattr(_KEEP, "tensors", None)
    if held is None:
        held = _KEEP.tensors = []
    if len(held) > 4096:                  # pointers taken outside a _check-wrapped call must not accumulate
        held.clear()
    held.append(t)
    return c_vp(t.data_ptr())


def _stream() -> c_vp:
    return c_vp(torch.cuda.current_stream().cuda_stream)


def _is_bf16(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float16:
        return 0
    raise TypeError(f"CUDA kernels take fp16 / bf16 activations, got {t.dtype}")


class Workspace:
    """Per-device scratch shared by kernels that need it: split-K partial tiles and their tile
    counters (GEMM), split-KV partials (attention) and the status word every bounded wait reports
    to.  Sized once; kernels fall back to un-split execution when a problem does not fit."""

    _by_device: Dict[int, "Workspace"] = {}

    def __init__(self, device: torch.device, gemm_bytes: int = 64 << 20, attn_floats: int = 32 << 20):
        self.gemm_ws = torch.empty(gemm_bytes, dtype=torch.uint8, device=device)
        self.counters = torch.zeros(8192, dtype=torch.int32, device=device)
        self.attn_ws = torch.empty(attn_floats, dtype=torch.float32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.argmax_keys = torch.zeros(256, dtype=torch.int64, device=device)
        self.argmax_counters = torch.zeros(256, dtype=torch.int32, device=device)

    @classmethod
    def get(cls, device: torch.device) -> "Workspace":
        idx = device.index if device.index is not None else torch.cuda.current_device()
        ws = cls._by_device.get(idx)
        if ws is None:
            ws = cls._by_device[idx] = Workspace(torch.device("cuda", idx))
        return ws

    def check_status(self) -> None:
        """Raise if any kernel recorded a timed-out wait (synchronises the device)."""
        code = int(self.status[0].item())
        if code != 0:
            self.status.zero_()
            names = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue", 4: "peer", 5: "bad argument"}
            raise RuntimeError(f"kernel wait timed out in role: {names.get(code, code)}")


# ------------------------------------------------------------------------------------------------


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.contiguous()
    y = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    _check(lib().telb_rmsnorm(_p(x), c_vp(0), _p(weight), _p(y), c_vp(0), c_ll(rows), c_int(x.shape[-1]), c_float(eps),
                              c_int(_is_bf16(x)), _stream()), "rmsnorm")
    return y


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    x = x.contiguous()
    residual = residual.contiguous()
    y = torch.empty_like(x)
    res = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    _check(lib().telb_rmsnorm(_p(x), _p(residual), _p(weight), _p(y), _p(res), c_ll(rows), c_int(x.shape[-1]),
                              c_float(eps), c_int(_is_bf16(x)), _stream()), "add_rmsnorm")
    return y, res


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    x = x.contiguous()
    y = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    _check(lib().telb_layernorm(_p(x), _p(weight), _p(bias), _p(y), c_ll(rows), c_int(x.shape[-1]), c_float(eps), c_int(_is_bf16(x)),
                                _stream()), "layernorm")
    return y


def gated_group_rmsnorm(x, z, weight, n_groups, eps):
    x, z = x.contiguous(), z.contiguous()
    y = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    _check(lib().telb_gated_group_rmsnorm(_p(x), _p(z), _p(weight), _p(y), c_ll(rows), c_int(x.shape[-1]),
                                          c_int(n_groups), c_float(eps), c_int(_is_bf16(x)), _stream()), "gated_group_rmsnorm")
    return y


def geglu(gate_up: torch.Tensor, tanh_approx: bool = True) -> torch.Tensor:
    rows, two = gate_up.shape
    inter = two // 2
    out = torch.empty(rows, inter, dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().telb_geglu(_p(gate_up), _p(out), c_ll(rows), c_int(inter), c_int(1 if tanh_approx else 0), c_int(_is_bf16(gate_up)),
                            _stream()), "geglu")
    return out


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    gate_up = gate_up.contiguous()
    inter = gate_up.shape[-1] // 2
    rows = gate_up.numel() // gate_up.shape[-1]
    out = torch.empty(*gate_up.shape[:-1], inter, dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().telb_swiglu(_p(gate_up), _p(out), c_ll(rows), c_int(inter), c_int(_is_bf16(gate_up)), _stream()), "swiglu")
    return out


def relu2(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous()
    out = torch.empty_like(x)
    _check(lib().telb_relu2(_p(x), _p(out), c_ll(x.numel()), c_int(_is_bf16(x)), _stream()), "relu2")
    return out


def gelu(x: torch.Tensor, tanh_approx: bool = False) -> torch.Tensor:
    x = x.contiguous()
    out = torch.empty_like(x)
    _check(lib().telb_gelu(_p(x), _p(out), c_ll(x.numel()), c_int(int(tanh_approx)), c_int(_is_bf16(x)), _stream()), "gelu")
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    ids = ids.to(torch.int32).contiguous()
    out = torch.empty(ids.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    _check(lib().telb_embedding(_p(ids), _p(table), _p(out), c_ll(ids.numel()), c_int(table.shape[1]),
                                c_int(table.shape[0]), c_int(_is_bf16(table)), _stream()), "embedding")
    return out


def embedding_quant(ids, data, scale, global_scale, fmt: str, out_dtype) -> torch.Tensor:
    """Gather rows of an FP8 (``data [V, H]`` E4M3, ``scale [V]`` fp32) or NVFP4 (``data [V, H / 2]``, ``scale [V, H / 16]`` E4M3,
    ``global_scale``) embedding table and expand them to ``out_dtype`` in the same kernel."""
    assert out_dtype in (torch.float16, torch.bfloat16) and fmt in ("fp8", "nvfp4")
    ids = ids.to(torch.int32).contiguous()
    hidden = data.shape[1] * (2 if fmt == "nvfp4" else 1)
    out = torch.empty(ids.numel(), hidden, dtype=out_dtype, device=data.device)
    d, sc = data.contiguous(), scale.contiguous()
    gs = None if global_scale is None else global_scale.reshape(-1).float().contiguous()
    _check(lib().telb_embedding_quant(_p(ids), _p(d), _p(sc), _p(gs), _p(out), c_ll(ids.numel()), c_int(hidden), c_int(data.shape[0]),
                                      c_int(1 if fmt == "nvfp4" else 0), c_int(int(out_dtype == torch.bfloat16)), _stream()), "embedding_quant")
    return out


def gemm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
         alpha: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, mode: int = 0, splits: int = 0) -> torch.Tensor:
    """``out[M,N] = x[M,K] · weight[N,K]ᵀ (* alpha[N]) (+ bias[N]) (+ residual[M,N])`` on tcgen05."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    m, k = x2.shape
    n = weight.shape[0]
    if weight.dtype != x.dtype:
        raise TypeError(f"gemm: activation {x.dtype} and weight {weight.dtype} differ")
    if k % 8:
        # rows must be 16-byte multiples for the TMA descriptors: zero columns up to the next multiple of 8 change nothing
        # (patch embeddings with 3 · 14 · 14 = 588 inputs are the case in practice; the padded copies are made per call)
        pad = 8 - k % 8
        x2 = torch.nn.functional.pad(x2, (0, pad))
        weight = torch.nn.functional.pad(weight, (0, pad))
        k += pad
    if out is None:
        out = torch.empty(m, n, dtype=x.dtype, device=x.device)
    ws = Workspace.get(x.device)
    _check(lib().telb_gemm_f16(_p(x2), _p(weight), _p(out), c_int(m), c_int(n), c_int(k), _p(bias), _p(alpha),
                               _p(residual), c_int(_is_bf16(x)), _p(ws.gemm_ws), c_ll(ws.gemm_ws.numel()),
                               _p(ws.counters), c_int(ws.counters.numel()), _p(ws.status), c_int(mode), c_int(splits),
                               _stream()), "gemm")
    return out.reshape(*lead, n)


def rope_table(inv_freq: torch.Tensor, attention_factor: float, max_pos: int, device) -> torch.Tensor:
    """``[max_pos, 2 * len(inv_freq)]`` fp32 cos | sin table from fp64 inverse frequencies, built on the device."""
    inv = inv_freq.to(device=device, dtype=torch.float64).contiguous()
    out = torch.empty(max_pos, 2 * inv.numel(), dtype=torch.float32, device=device)
    with torch.cuda.device(out.device):
        _check(lib().telb_rope_table(_p(inv), c_float(float(attention_factor)), _p(out), c_int(max_pos), c_int(inv.numel()), _stream()), "rope_table")
    return out


def mrope_rows(cos_sin: torch.Tensor, positions3: torch.Tensor, sections) -> torch.Tensor:
    """Per-row multimodal RoPE tables ``[T, D]`` gathered from the ordinary table by (temporal, height, width) positions."""
    half = cos_sin.shape[-1] // 2
    if len(sections) != 3 or sum(sections) != half:
        raise ValueError(f"mrope sections {list(sections)} must be three counts summing to {half}")
    cs = cos_sin.float().contiguous()
    p3 = positions3.to(device=cs.device, dtype=torch.int32).contiguous()
    out = torch.empty(p3.shape[1], 2 * half, dtype=torch.float32, device=cs.device)
    _check(lib().telb_mrope_rows(_p(cs), _p(p3), _p(out), c_int(p3.shape[1]), c_int(half), c_int(cs.shape[0]), c_int(int(sections[0])),
                                 c_int(int(sections[1])), _stream()), "mrope_rows")
    return out


def rope_kv_write(qkv, kv_layer, meta: StepMeta, cos_sin, num_q_heads, num_kv_heads, head_dim,
                  q_norm_w=None, k_norm_w=None, eps=1e-6) -> torch.Tensor:
    qkv = qkv.contiguous()
    t = qkv.shape[0]
    q = torch.empty(t, num_q_heads, head_dim, dtype=qkv.dtype, device=qkv.device)
    assert kv_layer.is_contiguous() and kv_layer.dtype == qkv.dtype
    positions = meta.positions
    if meta.rope_rows is not None:          # multimodal RoPE: per-row cos / sin tables prepared by the model
        cos_sin, positions = meta.rope_rows, meta.rope_pos
    _check(lib().telb_rope_kv_write(
        _p(qkv), _p(q), _p(kv_layer), _p(cos_sin), _p(positions), _p(meta.seq_ids), _p(meta.q_start),
        _p(meta.past_len), _p(meta.page_table), _p(meta.kv_offsets), _p(q_norm_w), _p(k_norm_w), c_int(t),
        c_int(num_q_heads), c_int(num_kv_heads), c_int(head_dim), c_int(cos_sin.shape[-1]), c_int(meta.page_size),
        c_int(meta.page_table.shape[1]), c_float(eps), c_int(_is_bf16(qkv)), _stream()), "rope_kv_write")
    return q


_KV_STAGE: Dict[tuple, torch.Tensor] = {}


def kv_fp8_stage(kv_layer: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The 16-bit staging layer an FP8 KV pool's attention works on (one per device, shape and type, shared by all layers)."""
    key = (kv_layer.device, tuple(kv_layer.shape), dtype)
    st = _KV_STAGE.get(key)
    if st is None:
        st = _KV_STAGE[key] = torch.zeros(kv_layer.shape, dtype=dtype, device=kv_layer.device)
    return st


def kv_fp8_load(kv_layer: torch.Tensor, stage: torch.Tensor, meta: StepMeta, scales: torch.Tensor, window: int = 0) -> None:
    """Expand the pages that hold the step's cached tokens from the FP8 layer ``[pages, 2, Hkv, P, D]`` into ``stage``."""
    _, _, hkv, psz, d = kv_layer.shape
    _check(lib().telb_kv_fp8_load(_p(kv_layer), _p(stage), _p(meta.past_len), _p(meta.page_table), _p(scales), c_int(meta.num_seqs),
                                  c_int(meta.page_table.shape[1]), c_int(psz), c_int(hkv), c_int(d), c_int(window or 0),
                                  c_int(_is_bf16(stage)), _stream()), "kv_fp8_load")


def kv_fp8_store(kv_layer: torch.Tensor, stage: torch.Tensor, meta: StepMeta, scales: torch.Tensor, q: Optional[torch.Tensor] = None):
    """Quantise the step's new K / V rows from ``stage`` into the FP8 layer and write the rounded values back to ``stage``.
    With ``q`` ``[T, Hq, D]`` the same launch also casts the query rows to E4M3 and returns them (else None)."""
    _, _, hkv, psz, d = kv_layer.shape
    q8 = None
    if q is not None:
        q = q.contiguous()
        q8 = torch.empty(q.shape, dtype=torch.float8_e4m3fn, device=q.device)
    _check(lib().telb_kv_fp8_store(_p(kv_layer), _p(stage), _p(meta.seq_ids), _p(meta.q_start), _p(meta.past_len), _p(meta.page_table),
                                   _p(meta.kv_offsets), _p(scales), c_int(meta.num_tokens), c_int(meta.page_table.shape[1]), c_int(psz),
                                   c_int(hkv), c_int(d), c_int(_is_bf16(stage)), _p(q), _p(q8), c_int(q.shape[1] if q is not None else 0),
                                   _stream()), "kv_fp8_store")
    return q8


def fp8_decode_ok(q_shape, hkv: int, meta: StepMeta) -> bool:
    """Whether the decode kernel that reads FP8 pages in place covers this step (decode-shaped, head_dim 128)."""
    t, hq, d = q_shape
    group = hq // hkv
    return (meta.tree_mask is None and d == 128 and meta.max_q_len * group <= 16 and 16 % group == 0
            and os.environ.get("TELB_DISABLE_FP8_DECODE_ATTN", "0") != "1")


def paged_attention_decode_fp8(q8: torch.Tensor, kv_layer: torch.Tensor, meta: StepMeta, scale: float, sliding_window, kv_scales: torch.Tensor,
                               out_dtype: torch.dtype, out_scale: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None,
                               splits: Optional[int] = None):
    """Decode-shaped attention over FP8 (E4M3) pages read in place.  ``q8``: the query rows cast to E4M3.  Returns 16-bit rows
    ``[T, Hq, D]`` of ``out_dtype``, or ``QuantActs`` over ``[T, Hq * D]`` when ``out_scale`` (the next projection's NVFP4 input
    scale) is given."""
    t, hq, d = q8.shape
    hkv = kv_layer.shape[2]
    if splits is None:
        splits = _decode_splits(meta, hkv)
    ws = Workspace.get(q8.device)
    L = lib()
    out = xq = sf = None
    if out_scale is None:
        out = torch.empty(t, hq, d, dtype=out_dtype, device=q8.device)
    else:
        L.telb_nvfp4_sf_bytes.restype = c_ll
        xq = torch.empty(t, hq * d // 2, dtype=torch.uint8, device=q8.device)
        sf = _sf_buffer(L.telb_nvfp4_sf_bytes(c_ll(t), c_int(hq * d)), hq * d, q8.device)
    if sinks is not None:
        sinks = sinks.to(device=q8.device, dtype=torch.float32).contiguous()
    _check(L.telb_paged_attention_decode_fp8(
        _p(q8), _p(kv_layer), _p(out), _p(xq), _p(sf), _p(out_scale), _p(kv_scales), _p(meta.q_start), _p(meta.q_len), _p(meta.past_len),
        _p(meta.page_table), c_int(meta.num_seqs), c_int(t), c_int(meta.max_q_len), c_int(kv_layer.shape[0]), c_int(meta.page_table.shape[1]),
        c_int(meta.page_size), c_int(hq), c_int(hkv), c_int(d), c_float(scale), c_int(sliding_window or 0), c_int(splits), _p(ws.attn_ws),
        c_ll(ws.attn_ws.numel()), c_int(1 if out_dtype == torch.bfloat16 else 0), _p(ws.status), _p(sinks), _stream()),
        "paged_attention_decode_fp8", 2 if splits > 1 else 1)
    return out if out_scale is None else QuantActs(xq, sf, (t, hq * d), out_dtype)


def _attn_splits(meta: StepMeta, hkv: int, group: int) -> int:
    tq = 128 // group
    qtiles = (meta.max_q_len + tq - 1) // tq
    ctas = meta.num_seqs * hkv * qtiles
    if ctas >= 148 or meta.max_q_len > 4 * tq:
        return 1
    kv_tiles = max(1, (meta.max_seq_len + 63) // 64)
    return max(1, min((2 * 148 + ctas - 1) // ctas, kv_tiles, 32))


def _decode_splits(meta: StepMeta, hkv: int) -> int:
    ctas = meta.num_seqs * hkv
    if ctas >= 148:
        return 1
    tiles = max(1, (meta.max_seq_len + 127) // 128)
    return max(1, min((148 + ctas - 1) // ctas, tiles, 32))


def paged_attention(q, kv_layer, meta: StepMeta, scale, sliding_window=None, sinks=None, splits: Optional[int] = None,
                    kernel: Optional[str] = None, trace: Optional[torch.Tensor] = None, causal: bool = True,
                    skip_thr: Optional[torch.Tensor] = None, skip_stats: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged GQA attention.  Decode-shaped steps (``max_q_len * Hq/Hkv <= 16``, head_dim 128, causal)
    run the token-major XQA-style kernel; everything else the row-major tile kernel.
    ``kernel`` forces ``"decode"`` or ``"tile"``; ``causal=False`` lets every row see every token of its sequence."""
    if not causal:
        sliding_window, kernel = -1, "tile"
    if sinks is not None:
        sinks = sinks.to(device=q.device, dtype=torch.float32).contiguous()
    q = q.contiguous()
    t, hq, d = q.shape
    hkv = kv_layer.shape[2]
    group = hq // hkv
    out = torch.empty_like(q)
    ws = Workspace.get(q.device)
    tm = meta.tree_mask
    decode_ok = (tm is None and d == 128 and meta.max_q_len * group <= 16 and 16 % group == 0)
    if skip_thr is None:
        skip_thr = meta.skip_thr            # per-sequence skip-softmax thresholds of the step (prefill-size steps only)
    if skip_thr is not None:
        skip_thr = skip_thr.to(device=q.device, dtype=torch.float32).contiguous()
        if kernel is None and meta.max_q_len * group > 16:
            kernel = "tile"
    use_decode = decode_ok if kernel is None else (kernel == "decode")
    if use_decode:
        if not decode_ok:
            raise ValueError("step is not decode-shaped")
        if splits is None:
            splits = _decode_splits(meta, hkv)
        _check(lib().telb_paged_attention_decode_traced(
            _p(q), _p(kv_layer), _p(out), _p(meta.q_start), _p(meta.q_len), _p(meta.past_len), _p(meta.page_table),
            c_int(meta.num_seqs), c_int(t), c_int(meta.max_q_len), c_int(kv_layer.shape[0]), c_int(meta.page_table.shape[1]),
            c_int(meta.page_size), c_int(hq), c_int(hkv), c_int(d), c_float(scale), c_int(sliding_window or 0), c_int(splits),
            _p(ws.attn_ws), c_ll(ws.attn_ws.numel()), c_int(_is_bf16(q)), _p(ws.status), _p(trace), _p(sinks), _stream()),
            "paged_attention_decode", 2 if splits > 1 else 1)
        return out
    if splits is None:
        splits = _attn_splits(meta, hkv, group)
    _check(lib().telb_paged_attention(
        _p(q), _p(kv_layer), _p(out), _p(meta.q_start), _p(meta.q_len), _p(meta.past_len), _p(meta.page_table),
        _p(tm), c_int(tm.shape[1] if tm is not None else 0), c_int(meta.num_seqs), c_int(t), c_int(meta.max_q_len),
        c_int(kv_layer.shape[0]), c_int(meta.page_table.shape[1]), c_int(meta.page_size), c_int(hq), c_int(hkv),
        c_int(d), c_float(scale), c_int(sliding_window or 0), c_int(splits), _p(ws.attn_ws), c_ll(ws.attn_ws.numel()),
        c_int(_is_bf16(q)), _p(ws.status), _p(sinks), _p(skip_thr), _p(skip_stats), _stream()), "paged_attention", 2 if splits > 1 else 1)
    return out


def decode_attention_quant_ok(q_shape, hkv: int, meta: StepMeta) -> bool:
    """Whether :func:`paged_attention_quant` covers this step (the decode-shaped kernel, head_dim 128)."""
    t, hq, d = q_shape
    group = hq // hkv
    return (meta.tree_mask is None and d == 128 and meta.max_q_len * group <= 16 and 16 % group == 0
            and os.environ.get("TELB_DISABLE_ATTN_QUANT_FUSION", "0") != "1")


def paged_attention_quant(q, kv_layer, meta: StepMeta, scale, sliding_window, out_scale: torch.Tensor,
                          splits: Optional[int] = None, sinks: Optional[torch.Tensor] = None) -> "QuantActs":
    """Decode-shaped paged attention whose epilogue (or split merge) writes NVFP4 rows ``[T, Hq * D]`` quantised with the
    global scale ``out_scale`` of the projection that follows, instead of 16-bit rows and a quantisation kernel."""
    q = q.contiguous()
    t, hq, d = q.shape
    hkv = kv_layer.shape[2]
    if not decode_attention_quant_ok(q.shape, hkv, meta):
        raise ValueError("step is not decode-shaped")
    if splits is None:
        splits = _decode_splits(meta, hkv)
    L = lib()
    L.telb_nvfp4_sf_bytes.restype = c_ll
    width = hq * d
    xq = torch.empty(t, width // 2, dtype=torch.uint8, device=q.device)
    sf = _sf_buffer(L.telb_nvfp4_sf_bytes(c_ll(t), c_int(width)), width, q.device)
    ws = Workspace.get(q.device)
    _check(L.telb_paged_attention_decode_quant(
        _p(q), _p(kv_layer), _p(xq), _p(sf), _p(out_scale), _p(meta.q_start), _p(meta.q_len), _p(meta.past_len), _p(meta.page_table),
        c_int(meta.num_seqs), c_int(t), c_int(meta.max_q_len), c_int(kv_layer.shape[0]), c_int(meta.page_table.shape[1]),
        c_int(meta.page_size), c_int(hq), c_int(hkv), c_int(d), c_float(scale), c_int(sliding_window or 0), c_int(splits),
        _p(ws.attn_ws), c_ll(ws.attn_ws.numel()), c_int(_is_bf16(q)), _p(ws.status),
        _p(None if sinks is None else sinks.to(device=q.device, dtype=torch.float32).contiguous()), _stream()),
        "paged_attention_decode_quant", 2 if splits > 1 else 1)
    return QuantActs(xq, sf, (t, width), q.dtype)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    assert logits.dim() == 2 and logits.stride(1) == 1
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    dt = 2 if logits.dtype == torch.float32 else _is_bf16(logits)
    ws = Workspace.get(logits.device)
    _check(lib().telb_argmax(_p(logits), _p(out), c_ll(logits.shape[0]), c_int(logits.shape[1]),
                             c_ll(logits.stride(0)), c_int(dt), _p(ws.argmax_keys), _p(ws.argmax_counters),
                             c_int(ws.argmax_keys.numel()), _stream()), "argmax")
    return out




# ---- NVFP4 -----------------------------------------------------------------------------------


def nvfp4_swizzle_scales(weight_scale: torch.Tensor) -> torch.Tensor:
    """Row-major E4M3 block scales ``[rows, K/16]`` → the 512-byte atom layout the tensor core reads
    (``[ceil(rows/128), K/64 padded to whole 256-element stages, 512]`` bytes)."""
    sf = weight_scale.view(torch.uint8).contiguous()
    rows, kb = sf.shape
    k = kb * 16
    L = lib()
    L.telb_nvfp4_sf_bytes.restype = c_ll
    nbytes = L.telb_nvfp4_sf_bytes(c_ll(rows), c_int(k))
    out = torch.empty(nbytes, dtype=torch.uint8, device=sf.device)
    _check(L.telb_nvfp4_swizzle_scales(_p(sf), _p(out), c_ll(rows), c_int(k), _stream()), "nvfp4_swizzle_scales")
    return out


class QuantActs:
    """Activations already quantised to NVFP4 by their producer (packed codes + atom-layout scales)."""

    __slots__ = ("xq", "sf", "shape", "dtype", "ag_wait")

    def __init__(self, xq: torch.Tensor, sf: torch.Tensor, shape, dtype):
        self.xq, self.sf, self.shape, self.dtype = xq, sf, tuple(shape), dtype
        self.ag_wait = None      # GemmFusion when the rows are still being gathered from peers

    @property
    def is_cuda(self) -> bool:
        return True


def _sf_buffer(nbytes: int, k: int, device) -> torch.Tensor:
    # Rows beyond M only feed accumulator rows that are never stored, so they may hold anything;
    # K padding multiplies real rows and must be zero.
    return (torch.zeros if k % 256 else torch.empty)(nbytes, dtype=torch.uint8, device=device)


def rmsnorm_quant(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                  global_scale: torch.Tensor):
    """``(residual add +) RMSNorm`` whose output is written as NVFP4 only.  Returns
    ``(QuantActs, new_residual)`` (``new_residual`` is ``x`` itself when there is no residual)."""
    x = x.contiguous()
    m, k = x.shape
    L = lib()
    L.telb_nvfp4_sf_bytes.restype = c_ll
    nbytes = L.telb_nvfp4_sf_bytes(c_ll(m), c_int(k))
    xq = torch.empty(m, k // 2, dtype=torch.uint8, device=x.device)
    sf = _sf_buffer(nbytes, k, x.device)
    res_out = torch.empty_like(x) if residual is not None else None
    _check(L.telb_rmsnorm_quant(_p(x), _p(residual), _p(weight), _p(res_out), c_vp(0), _p(xq), _p(sf), _p(global_scale),
                                c_ll(m), c_int(k), c_float(eps), c_int(_is_bf16(x)), _stream()), "rmsnorm_quant")
    return QuantActs(xq, sf, (m, k), x.dtype), (res_out if residual is not None else x)


def gemm_nvfp4_swiglu(x: "QuantActs", weight: torch.Tensor, w_sf: torch.Tensor, alpha: torch.Tensor, out_scale: torch.Tensor,
                      fusion=None) -> "QuantActs":
    """Gate/up projection whose epilogue applies SwiGLU and quantises to NVFP4: ``weight [2·I, K/2]`` holds blocks of 64
    gate rows alternating with their up rows; returns the quantised ``[M, I]`` activations (M > 128)."""
    m, n, k = x.xq.shape[0], weight.shape[0], x.xq.shape[1] * 2
    inter = n // 2
    L = lib()
    L.telb_nvfp4_sf_bytes.restype = c_ll
    xq = torch.empty(m, inter // 2, dtype=torch.uint8, device=weight.device)
    sf = _sf_buffer(L.telb_nvfp4_sf_bytes(c_ll(m), c_int(inter)), inter, weight.device)
    ws = Workspace.get(weight.device)
    _check(L.telb_gemm_nvfp4_swiglu(_p(x.xq), _p(x.sf), _p(weight), _p(w_sf), _p(alpha), _p(xq), _p(sf), _p(out_scale), c_int(m), c_int(n),
                                    c_int(k), c_int(1 if x.dtype == torch.bfloat16 else 0), _p(ws.status),
                                    ctypes.byref(fusion) if fusion is not None else c_vp(0), _stream()), "gemm_nvfp4_swiglu")
    return QuantActs(xq, sf, (m, inter), x.dtype)


def gemm_skinny_swiglu(x: "QuantActs", weight: torch.Tensor, w_sf: torch.Tensor, alpha: torch.Tensor, out_scale: torch.Tensor,
                       fusion=None) -> "QuantActs":
    """Decode-size form of :func:`gemm_nvfp4_swiglu` (M <= 64): the swapped-operand, cluster split-K kernel applies SwiGLU and
    quantises in its epilogue, so a decode step has no separate activation kernel between the gate/up and down projections."""
    m, n, k = x.xq.shape[0], weight.shape[0], x.xq.shape[1] * 2
    inter = n // 2
    L = lib()
    L.telb_nvfp4_sf_bytes.restype = c_ll
    xq = torch.empty(m, inter // 2, dtype=torch.uint8, device=weight.device)
    sf = _sf_buffer(L.telb_nvfp4_sf_bytes(c_ll(m), c_int(inter)), inter, weight.device)
    ws = Workspace.get(weight.device)
    _check(L.telb_gemm_skinny_swiglu(c_int(1), _p(x.xq), _p(x.sf), _p(weight), _p(w_sf), _p(alpha), _p(xq), _p(sf), _p(out_scale), c_int(m),
                                     c_int(n), c_int(k), c_int(1 if x.dtype == torch.bfloat16 else 0), _p(ws.status),
                                     ctypes.byref(fusion) if fusion is not None else c_vp(0), _stream()), "gemm_skinny_swiglu")
    return QuantActs(xq, sf, (m, inter), x.dtype)


def swiglu_quant(gate_up: torch.Tensor, global_scale: torch.Tensor, interleaved: bool = False, moe_ws=None) -> QuantActs:
    """``moe_ws``: the routing tables of a grouped (mixture-of-experts) buffer; its padding rows are skipped."""
    gate_up = gate_up.contiguous()
    m = gate_up.shape[0]
    inter = gate_up.shape[1] // 2
    L = lib()
    L.telb_nvfp4_sf_bytes.restype = c_ll
    nbytes = L.telb_nvfp4_sf_bytes(c_ll(m), c_int(inter))
    xq = torch.empty(m, inter // 2, dtype=torch.uint8, device=gate_up.device)
    sf = _sf_buffer(nbytes, inter, gate_up.device)
    tile_rows = c_vp(moe_ws.tile_expert.data_ptr() + 4 * moe_ws.max_tiles) if moe_ws is not None else c_vp(0)
    _check(L.telb_swiglu_quant_rows(_p(gate_up), _p(xq), _p(sf), _p(global_scale), c_ll(m), c_int(inter),
                                    c_int(_is_bf16(gate_up)), c_int(1 if interleaved else 0), tile_rows, _stream()), "swiglu_quant")
    return QuantActs(xq, sf, (m, inter), gate_up.dtype)


def nvfp4_quantize(x: torch.Tensor, global_scale: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise activations ``[M,K]`` to packed E2M1 ``[M,K/2]`` + atom-layout E4M3 scales."""
    x = x.contiguous()
    m, k = x.shape
    L = lib()
    L.telb_nvfp4_sf_bytes.restype = c_ll
    nbytes = L.telb_nvfp4_sf_bytes(c_ll(m), c_int(k))
    xq = torch.empty(m, k // 2, dtype=torch.uint8, device=x.device)
    sf = _sf_buffer(nbytes, k, x.device)
    _check(L.telb_nvfp4_quantize(_p(x), _p(xq), _p(sf), _p(global_scale), c_ll(m), c_int(k), c_int(_is_bf16(x)), _stream()),
           "nvfp4_quantize")
    return xq, sf


def gemm_nvfp4(xq, x_sf, wq, w_sf, alpha, out_dtype, bias=None, residual=None, mode: int = 0, splits: int = 0):
    m, n, k = xq.shape[0], wq.shape[0], xq.shape[1] * 2
    out = torch.empty(m, n, dtype=out_dtype, device=xq.device)
    ws = Workspace.get(xq.device)
    _check(lib().telb_gemm_nvfp4(_p(xq), _p(x_sf), _p(wq), _p(w_sf), _p(out), c_int(m), c_int(n), c_int(k), _p(alpha),
                                 _p(bias), _p(residual), c_int(1 if out_dtype == torch.bfloat16 else 0), _p(ws.gemm_ws),
                                 c_ll(ws.gemm_ws.numel()), _p(ws.counters), c_int(ws.counters.numel()), _p(ws.status),
                                 c_int(mode), c_int(splits), _stream()), "gemm_nvfp4")
    return out


def nvfp4_linear(x, weight, weight_sf_atoms, alpha, input_scale, bias=None, quantize_activations=True):
    """NVFP4 linear: dynamic per-16 activation quantisation (calibrated global scale) + block-scaled GEMM."""
    if not quantize_activations:
        raise NotImplementedError("W4A16 NVFP4 runs through the W4A4 tensor-core path only when activations are quantised")
    if isinstance(x, QuantActs):
        return gemm_nvfp4(x.xq, x.sf, weight, weight_sf_atoms, alpha, x.dtype, bias)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    xq, x_sf = nvfp4_quantize(x2, input_scale)
    out = gemm_nvfp4(xq, x_sf, weight, weight_sf_atoms, alpha, x.dtype, bias)
    return out.reshape(*lead, weight.shape[0])


class GemmFusion(ctypes.Structure):
    """Host mirror of ``TelbGemmFusion`` (``csrc/kernels/gemm_common.cuh``)."""
    _fields_ = [("rs_out", c_vp * 8), ("rs_world", c_int), ("rs_rank", c_int), ("rs_rows_per_rank", c_int), ("pad0", c_int),
                ("ag_flags", c_vp), ("ag_epoch", c_vp), ("ag_world", c_int), ("ag_rows_per_rank", c_int)]


def gemm_fused(x, weight, fusion: GemmFusion, *, w_sf=None, alpha=None, bias=None, out=None, out_dtype=None):
    """Large-M GEMM with a fused tensor-parallel collective: ``x`` is 16-bit ``[M, K]`` or ``QuantActs``.
    With a reduce-scatter epilogue the rows land in the peers' partial buffers and nothing is returned."""
    ws = Workspace.get(weight.device)
    scatter = fusion.rs_world > 1
    if isinstance(x, QuantActs):
        m, n, k = x.xq.shape[0], weight.shape[0], x.xq.shape[1] * 2
        dt = out_dtype or x.dtype
        if out is None and not scatter:
            out = torch.empty(m, n, dtype=dt, device=weight.device)
        _check(lib().telb_gemm_nvfp4_fused(_p(x.xq), _p(x.sf), _p(weight), _p(w_sf), _p(out), c_int(m), c_int(n), c_int(k), _p(alpha),
                                           _p(bias), c_int(1 if dt == torch.bfloat16 else 0), _p(ws.status), ctypes.byref(fusion),
                                           _stream()), "gemm_nvfp4_fused")
        return out
    m, k = x.shape
    n = weight.shape[0]
    if out is None and not scatter:
        out = torch.empty(m, n, dtype=x.dtype, device=x.device)
    _check(lib().telb_gemm_f16_fused(_p(x), _p(weight), _p(out), c_int(m), c_int(n), c_int(k), _p(bias), _p(alpha), c_int(_is_bf16(x)),
                                     _p(ws.status), ctypes.byref(fusion), _stream()), "gemm_f16_fused")
    return out


def gemm_skinny(x, weight, *, x_sf=None, w_sf=None, alpha=None, bias=None, residual=None, out_dtype=None, ranks: int = 0):
    """Decode-size GEMM (M <= 128) with an explicit cluster size (``ranks`` K-slices; 0 = choose).
    16-bit operands when no scale tensors are given, NVFP4 otherwise."""
    kind = 1 if w_sf is not None else 0
    m = x.shape[0]
    n = weight.shape[0]
    k = x.shape[1] * (2 if kind else 1)
    dt = out_dtype or x.dtype
    out = torch.empty(m, n, dtype=dt, device=x.device)
    ws = Workspace.get(x.device)
    _check(lib().telb_gemm_skinny(c_int(kind), _p(x), _p(x_sf), _p(weight), _p(w_sf), _p(out), c_int(m), c_int(n), c_int(k),
                                  _p(alpha), _p(bias), _p(residual), c_int(1 if dt == torch.bfloat16 else 0), _p(ws.status),
                                  c_int(ranks), _stream()), "gemm_skinny")
    return out


INT4_GEMV_MAX_ROWS = 0 if os.environ.get("TELB_DISABLE_INT4_GEMV", "0") == "1" else 4


def gemm_int4_awq(x: torch.Tensor, wq: torch.Tensor, scales: torch.Tensor, group: int, bias=None, residual=None, ranks: int = 0):
    """W4A16 linear on ModelOpt-prepacked INT4 weights (``wq [N/2, K]`` uint8, ``scales [N, K/group]`` in ``x``'s dtype).
    Decode-size steps (M <= 128) expand the 4-bit tiles inside the GEMM kernel, so only 4-bit weights cross HBM; larger
    steps expand the matrix once into a temporary and run the dense tensor-core GEMM (compute-bound there)."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    m, k = x2.shape
    n = wq.shape[0] * 2
    if scales.dtype != x.dtype:
        scales = scales.to(x.dtype)
    ok = n % 2 == 0 and k % 64 == 0 and group >= 64 and group % 64 == 0 and k % group == 0
    if m <= INT4_GEMV_MAX_ROWS and ok and m * k * 2 <= 200 * 1024:
        # one to four rows: a CUDA-core GEMV streams the packed weights once (the tensor-core tile would be almost empty)
        out = torch.empty(m, n, dtype=x.dtype, device=x.device)
        _check(lib().telb_gemv_int4(_p(x2), _p(wq), _p(scales.contiguous()), _p(out), c_int(m), c_int(n), c_int(k), c_int(group), _p(bias),
                                    _p(residual.reshape(m, n).contiguous() if residual is not None else None), c_int(_is_bf16(x)), _stream()),
               "gemv_int4")
        return out.reshape(*lead, n)
    if m <= 128 and ok:
        out = torch.empty(m, n, dtype=x.dtype, device=x.device)
        ws = Workspace.get(x.device)
        _check(lib().telb_gemm_skinny_int4(_p(x2), _p(wq), _p(scales.contiguous()), _p(out), c_int(m), c_int(n), c_int(k), c_int(group), _p(bias),
                                           _p(residual), c_int(_is_bf16(x)), _p(ws.status), c_int(ranks), _stream()), "gemm_skinny_int4")
        return out.reshape(*lead, n)
    dense = torch.empty(n, k, dtype=x.dtype, device=x.device)
    _check(lib().telb_int4_awq_expand(_p(wq), _p(scales.contiguous()), _p(dense), c_int(n), c_int(k), c_int(group), c_int(_is_bf16(x)), _stream()),
           "int4_awq_expand")
    return gemm(x2, dense, bias=bias, residual=residual).reshape(*lead, n)


# ---- sampling ----------------------------------------------------------------------------------


def _logit_dtype(t: torch.Tensor) -> int:
    return 2 if t.dtype == torch.float32 else _is_bf16(t)


def sample(logits, temperature, top_k, top_p, uniforms) -> torch.Tensor:
    assert logits.dim() == 2 and logits.stride(1) == 1
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(lib().telb_sample(_p(logits), c_ll(logits.stride(0)), c_int(rows), c_int(vocab),
                             _p(temperature.to(torch.float32).contiguous()), _p(top_k.to(torch.int32).contiguous()),
                             _p(top_p.to(torch.float32).contiguous()), _p(uniforms.to(torch.float32).contiguous()), _p(out),
                             c_int(_logit_dtype(logits)), _stream()), "sample")
    return out


def token_logprobs(logits, tokens, k: int):
    """``(chosen [rows] fp32, top_ids [rows, k] int32, top_values [rows, k] fp32)``: log-probability of ``tokens[row]`` and the ``k``
    most likely tokens of every row under ``softmax(logits[row])``."""
    assert logits.dim() == 2 and logits.stride(1) == 1 and 0 <= k <= 32
    rows, vocab = logits.shape
    tok = tokens.to(device=logits.device, dtype=torch.int32).contiguous()
    chosen = torch.empty(rows, dtype=torch.float32, device=logits.device)
    ids = torch.empty(rows, max(k, 1), dtype=torch.int32, device=logits.device)
    vals = torch.empty(rows, max(k, 1), dtype=torch.float32, device=logits.device)
    _check(lib().telb_token_logprobs(_p(logits), c_ll(logits.stride(0)), c_int(rows), c_int(vocab), _p(tok), c_int(k), _p(chosen), _p(ids),
                                     _p(vals), c_int(_logit_dtype(logits)), _stream()), "token_logprobs")
    return chosen, ids[:, :k], vals[:, :k]


def apply_token_bitmask(logits: torch.Tensor, bitmask: torch.Tensor) -> torch.Tensor:
    """In place: entries whose bit is 0 in ``bitmask [rows, ceil(V/32)]`` become very negative."""
    _check(lib().telb_apply_token_bitmask(_p(logits), c_ll(logits.stride(0)), c_int(logits.shape[0]), c_int(logits.shape[1]),
                                          _p(bitmask.to(torch.int32).contiguous()), c_int(_logit_dtype(logits)), _stream()),
           "apply_token_bitmask")
    return logits


# ---- mixture of experts -------------------------------------------------------------------------


def moe_route_softmax_topk(logits, top_k, renormalize=True, bias=None, sigmoid=False, n_group=1, topk_group=1,
                           scaling=1.0):
    logits = logits.contiguous()
    t, e = logits.shape
    w = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    idx = torch.empty(t, top_k, dtype=torch.int32, device=logits.device)
    _check(lib().telb_moe_route(_p(logits), _p(w), _p(idx), _p(bias.float().contiguous() if bias is not None else None), c_int(t), c_int(e), c_int(top_k), c_int(int(renormalize)),
                                c_int(int(sigmoid)), c_int(n_group), c_int(topk_group), c_float(scaling), c_int(_logit_dtype(logits)),
                                _stream()), "moe_route")
    return w, idx


class MoeWorkspace:
    """Routing tables of one MoE call over the padded row space (every expert segment is a multiple
    of 128 rows, so a 128-row tile belongs to exactly one expert)."""

    def __init__(self, tokens: int, top_k: int, experts_local: int, device):
        slots = tokens * top_k
        self.max_tiles = (slots + 127) // 128 + experts_local
        self.rows_pad = self.max_tiles * 128
        self.dst_row = torch.empty(slots, dtype=torch.int32, device=device)
        # [0, max_tiles): expert of each 128-row tile (-1 = unused); [max_tiles, 2 max_tiles): rows in use in each tile
        self.tile_expert = torch.empty(2 * self.max_tiles, dtype=torch.int32, device=device)
        self.counts = torch.empty(1, dtype=torch.int32, device=device)


def moe_align(topk_idx: torch.Tensor, experts: int, expert_lo: int, expert_hi: int) -> MoeWorkspace:
    t, k = topk_idx.shape
    ws = MoeWorkspace(t, k, expert_hi - expert_lo, topk_idx.device)
    _check(lib().telb_moe_align(_p(topk_idx), _p(ws.dst_row), _p(ws.tile_expert), _p(ws.counts), c_int(t * k), c_int(experts),
                                c_int(expert_lo), c_int(expert_hi), c_int(ws.max_tiles), _stream()), "moe_align")
    return ws


def moe_gather(x: torch.Tensor, ws: MoeWorkspace, top_k: int, quant_scale: Optional[torch.Tensor]):
    """Routed rows in expert order: NVFP4 ``QuantActs`` when ``quant_scale`` is given, else 16-bit."""
    x = x.contiguous()
    t, h = x.shape
    if quant_scale is None:
        out = torch.empty(ws.rows_pad, h, dtype=x.dtype, device=x.device)
        _check(lib().telb_moe_gather(_p(x), _p(ws.dst_row), _p(out), c_vp(0), c_vp(0), c_vp(0), c_int(t * top_k), c_int(top_k),
                                     c_int(h), c_int(_is_bf16(x)), _stream()), "moe_gather")
        return out
    L = lib()
    L.telb_nvfp4_sf_bytes.restype = c_ll
    xq = torch.empty(ws.rows_pad, h // 2, dtype=torch.uint8, device=x.device)
    sf = _sf_buffer(L.telb_nvfp4_sf_bytes(c_ll(ws.rows_pad), c_int(h)), h, x.device)
    _check(L.telb_moe_gather(_p(x), _p(ws.dst_row), c_vp(0), _p(xq), _p(sf), _p(quant_scale), c_int(t * top_k), c_int(top_k),
                             c_int(h), c_int(_is_bf16(x)), _stream()), "moe_gather")
    return QuantActs(xq, sf, (ws.rows_pad, h), x.dtype)


def gemm_grouped(x, weight, ws: MoeWorkspace, experts_local: int, alpha=None, bias=None, w_sf=None):
    """Expert GEMM over the padded rows: ``x`` 16-bit ``[rows_pad, K]`` or ``QuantActs``; ``weight``
    ``[E_local * N, K]`` (16-bit) or packed NVFP4 ``[E_local * N, K/2]`` with atom scales ``w_sf``."""
    wsx = Workspace.get(weight.device)
    if isinstance(x, QuantActs):
        n = weight.shape[0] // experts_local
        k = weight.shape[1] * 2
        out = torch.empty(ws.rows_pad, n, dtype=x.dtype, device=weight.device)
        _check(lib().telb_gemm_nvfp4_grouped(_p(x.xq), _p(x.sf), _p(weight), _p(w_sf), _p(out), c_int(ws.rows_pad), c_int(n), c_int(k),
                                             c_int(experts_local), _p(ws.tile_expert), _p(alpha),
                                             c_int(1 if x.dtype == torch.bfloat16 else 0), _p(wsx.status), _stream()),
               "gemm_nvfp4_grouped")
        return out
    n = weight.shape[0] // experts_local
    k = weight.shape[1]
    out = torch.empty(ws.rows_pad, n, dtype=x.dtype, device=x.device)
    _check(lib().telb_gemm_f16_grouped(_p(x), _p(weight), _p(out), c_int(ws.rows_pad), c_int(n), c_int(k), c_int(experts_local),
                                       _p(ws.tile_expert), _p(alpha), _p(bias), c_int(_is_bf16(x)), _p(wsx.status), _stream()),
           "gemm_f16_grouped")
    return out


def gemm_grouped_swiglu(x: "QuantActs", weight, ws: MoeWorkspace, experts_local: int, alpha, w_sf, out_scale: torch.Tensor) -> "QuantActs":
    """Expert gate/up GEMM over the padded rows whose epilogue applies SwiGLU and quantises to NVFP4 for the second expert GEMM
    (each expert's ``2 * inter`` weight rows alternate gate / up in blocks of 64).  Padding rows are left unwritten."""
    n = weight.shape[0] // experts_local
    k = weight.shape[1] * 2
    inter = n // 2
    L = lib()
    L.telb_nvfp4_sf_bytes.restype = c_ll
    xq = torch.empty(ws.rows_pad, inter // 2, dtype=torch.uint8, device=weight.device)
    sf = _sf_buffer(L.telb_nvfp4_sf_bytes(c_ll(ws.rows_pad), c_int(inter)), inter, weight.device)
    wsx = Workspace.get(weight.device)
    _check(L.telb_gemm_nvfp4_grouped_swiglu(_p(x.xq), _p(x.sf), _p(weight), _p(w_sf), _p(xq), _p(sf), _p(out_scale), c_int(ws.rows_pad),
                                            c_int(n), c_int(k), c_int(experts_local), _p(ws.tile_expert), _p(alpha),
                                            c_int(1 if x.dtype == torch.bfloat16 else 0), _p(wsx.status), _stream()),
           "gemm_nvfp4_grouped_swiglu")
    return QuantActs(xq, sf, (ws.rows_pad, inter), x.dtype)


def moe_combine(y: torch.Tensor, ws, topk_w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = Σ_k w[t,k] · y[ws.dst_row[t*K + k]]`` (slots with a negative row contribute nothing)."""
    t, k = topk_w.shape
    if out is None:
        out = torch.empty(t, y.shape[1], dtype=y.dtype, device=y.device)
    _check(lib().telb_moe_combine(_p(y), _p(ws.dst_row), _p(topk_w), _p(out), c_int(t), c_int(k), c_int(y.shape[1]),
                                  c_int(_is_bf16(y)), _stream()), "moe_combine")
    return out


# ---- recurrent layers ---------------------------------------------------------------------------


def causal_conv1d(x, weight, bias, conv_state, meta: StepMeta, activation=True):
    x = x.contiguous()
    t, c = x.shape
    w = weight.reshape(c, -1).contiguous()
    out = torch.empty_like(x)
    assert conv_state.is_contiguous() and conv_state.dtype == x.dtype
    _check(lib().telb_causal_conv1d(_p(x), _p(w), _p(bias), _p(conv_state), _p(out), _p(meta.seq_ids), _p(meta.q_start),
                                    _p(meta.q_len), _p(meta.past_len), _p(meta.slot_ids), c_int(t), c_int(meta.num_seqs), c_int(c),
                                    c_int(w.shape[1]), c_int(int(activation)), c_int(_is_bf16(x)), _stream()), "causal_conv1d", 2)
    return out


_SSM_SCRATCH = {}


SSD_TC_MIN_Q = 64        # steps whose longest sequence has at least this many new rows take the tensor-core chunk scan


def ssm_scan(x, dt, A, B, C, D, dt_bias, ssm_state, meta: StepMeta, z=None, dt_softplus=True, dt_limit=0.0):
    x, dt, B, C = x.contiguous(), dt.contiguous(), B.contiguous(), C.contiguous()
    t, nh, hd = x.shape
    y = torch.empty_like(x)
    assert ssm_state.dtype == torch.float32 and ssm_state.is_contiguous()
    if (meta.max_q_len >= SSD_TC_MIN_Q and hd == 64 and B.shape[-1] == 128 and os.environ.get("TELB_DISABLE_SSD_TC", "0") != "1"):
        # prefill: chunked state-space-duality scan on the tensor cores (csrc/kernels/ssd_tc5.cu)
        ws = Workspace.get(x.device)
        _check(lib().telb_ssd_chunk_scan(_p(x), _p(dt), _p(A.float().contiguous()), _p(B), _p(C), _p(D.float().contiguous()),
                                         _p(dt_bias.float().contiguous()), _p(z.contiguous() if z is not None else None), _p(ssm_state), _p(y),
                                         _p(meta.q_start), _p(meta.q_len), _p(meta.past_len), _p(meta.slot_ids), c_int(meta.num_seqs), c_int(t),
                                         c_int(nh), c_int(hd), c_int(B.shape[-1]), c_int(B.shape[1]), c_int(int(dt_softplus)),
                                         c_float(dt_limit), c_int(_is_bf16(x)), _p(ws.status), _stream()), "ssd_chunk_scan")
        return y
    scratch = None
    if meta.max_q_len >= 256:       # long prefill chunk: parallel segments need per-segment states (see recurrent.cu)
        segs = (meta.max_q_len + 127) // 128
        need = meta.num_seqs * nh * segs * (hd * B.shape[-1] + 1)
        scratch = _SSM_SCRATCH.get(x.device)
        if scratch is None or scratch.numel() < need:
            scratch = _SSM_SCRATCH[x.device] = torch.empty(need, dtype=torch.float32, device=x.device)
    _check(lib().telb_ssm_scan(_p(x), _p(dt), _p(A.float().contiguous()), _p(B), _p(C), _p(D.float().contiguous()),
                               _p(dt_bias.float().contiguous()), _p(z.contiguous() if z is not None else None), _p(ssm_state), _p(y),
                               _p(meta.q_start), _p(meta.q_len), _p(meta.past_len), _p(meta.slot_ids), c_int(meta.num_seqs),
                               c_int(nh), c_int(hd), c_int(B.shape[-1]), c_int(B.shape[1]), c_int(int(dt_softplus)),
                               c_float(dt_limit), c_int(_is_bf16(x)), c_int(meta.max_q_len), _p(scratch),
                               c_ll(scratch.numel() if scratch is not None else 0), _stream()), "ssm_scan", 3 if scratch is not None else 1)
    return y


GDN_TC_MIN_Q = 32        # steps whose longest sequence has at least this many new rows take the tensor-core chunked kernel


def gated_delta_rule(q, k, v, a, b, A_log, dt_bias, state, meta: StepMeta):
    q, k, v, a, b = (t.contiguous() for t in (q, k, v, a, b))
    out = torch.empty_like(v)
    assert state.dtype == torch.float32 and state.is_contiguous()
    if (meta.max_q_len >= GDN_TC_MIN_Q and q.shape[2] == 128 and v.shape[2] == 128 and os.environ.get("TELB_DISABLE_GDN_TC", "0") != "1"):
        # prefill: chunked (64-token) delta rule with the matrix products on the tensor cores (csrc/kernels/gdn_tc5.cu)
        ws = Workspace.get(q.device)
        _check(lib().telb_gdn_chunk_prefill(_p(q), _p(k), _p(v), _p(a), _p(b), _p(A_log.float().contiguous()), _p(dt_bias.float().contiguous()),
                                            _p(state), _p(out), _p(meta.q_start), _p(meta.q_len), _p(meta.past_len), _p(meta.slot_ids),
                                            c_int(meta.num_seqs), c_int(q.shape[0]), c_int(q.shape[1]), c_int(v.shape[1]), c_int(q.shape[2]),
                                            c_int(v.shape[2]), c_int(_is_bf16(q)), _p(ws.status), _stream()), "gdn_chunk_prefill")
        return out
    _check(lib().telb_gated_delta_rule(_p(q), _p(k), _p(v), _p(a), _p(b), _p(A_log.float().contiguous()),
                                       _p(dt_bias.float().contiguous()), _p(state), _p(out), _p(meta.q_start), _p(meta.q_len),
                                       _p(meta.past_len), _p(meta.slot_ids), c_int(meta.num_seqs), c_int(q.shape[1]), c_int(v.shape[1]),
                                       c_int(q.shape[2]), c_int(v.shape[2]), c_int(_is_bf16(q)), _stream()), "gated_delta_rule")
    return out


# ---- speculative decoding -------------------------------------------------------------------------


def spec_accept_greedy(target_tokens, tree_tokens, parents, max_path: int, force_len=0):
    b, n = tree_tokens.shape
    dev = tree_tokens.device
    force = None
    if isinstance(force_len, torch.Tensor):
        force = force_len.to(device=dev, dtype=torch.int32).contiguous()
    elif force_len:
        force = torch.full((b,), int(force_len), dtype=torch.int32, device=dev)
    path = torch.zeros(b, max_path, dtype=torch.int32, device=dev)
    plen = torch.empty(b, dtype=torch.int32, device=dev)
    bonus = torch.empty(b, dtype=torch.int32, device=dev)
    tt, tr, pa = target_tokens.to(torch.int32).contiguous(), tree_tokens.to(torch.int32).contiguous(), parents.to(torch.int32).contiguous()
    _check(lib().telb_spec_accept_greedy(_p(tt), _p(tr), _p(pa), _p(path), _p(plen), _p(bonus), c_int(b), c_int(n),
                                         c_int(max_path), _p(force), _stream()), "spec_accept_greedy")
    return path, plen, bonus


def eagle_tree_meta(parents: torch.Tensor, base_pos: torch.Tensor, depth_base: int, pos_offset: int):
    """Packed ancestor mask ``[B * R, ceil(R / 32)]``, depths ``[B, R]`` and positions ``[B * R]`` of a batch of trees given as
    parent tables ``[B, R]`` (parents precede children, ``-1`` = none): one kernel, nothing read back."""
    b, r = parents.shape
    dev = parents.device
    words = (r + 31) // 32
    par = parents.to(torch.int32).contiguous()
    mask = torch.empty(b * r, words, dtype=torch.int32, device=dev)
    depth = torch.empty(b, r, dtype=torch.int32, device=dev)
    pos = torch.empty(b * r, dtype=torch.int32, device=dev)
    base = base_pos.to(device=dev, dtype=torch.int32).contiguous()
    _check(lib().telb_eagle_tree_meta(_p(par), _p(base), _p(mask), _p(depth), _p(pos),
                                      c_int(b), c_int(r), c_int(words), c_int(depth_base), c_int(pos_offset), _stream()), "eagle_tree_meta")
    return mask, depth, pos


def eagle_select_verify(p_sc, p_tok, p_par, p_dep, root, keep: int):
    """The ``keep`` best candidates of each sequence's pool ``[B, P]`` in pool order behind the root: tokens, parents (indices into
    the tree, root = -1 for slot 0) and depths, each ``[B, keep + 1]`` int32."""
    b, pool = p_sc.shape
    dev = p_sc.device
    i32 = lambda t: t.to(device=dev, dtype=torch.int32).contiguous()
    # converted copies stay referenced until the launch: a temporary freed after its pointer was taken would hand its
    # memory to the next conversion
    sc, ptok, ppar, pdep, rt = p_sc.float().contiguous(), i32(p_tok), i32(p_par), i32(p_dep), i32(root)
    tok = torch.empty(b, keep + 1, dtype=torch.int32, device=dev)
    par = torch.empty_like(tok)
    dep = torch.empty_like(tok)
    _check(lib().telb_eagle_select_verify(_p(sc), _p(ptok), _p(ppar), _p(pdep), _p(rt),
                                          c_int(b), c_int(pool), c_int(keep), _p(tok), _p(par), _p(dep), _stream()), "eagle_select_verify")
    return tok, par, dep


def dflash2_grouped_dynamic_conv(hidden, delta, base, residual, block: int, group_size: int):
    """One side of DFlash 2's dynamic grouped convolution over whole proposal blocks (16-bit in, 16-bit out)."""
    assert hidden.dtype in (torch.float16, torch.bfloat16)
    h, d, b = hidden.contiguous(), delta.to(hidden.dtype).contiguous(), base.to(hidden.dtype).contiguous()
    r = None if residual is None else residual.to(hidden.dtype).contiguous()
    out = torch.empty_like(h)
    _check(lib().telb_dflash2_conv(_p(h), _p(d), _p(b), _p(r), _p(out), c_int(h.shape[0]), c_int(h.shape[1]), c_int(block),
                                   c_int(b.shape[0]), c_int(group_size), c_int(int(h.dtype == torch.bfloat16)), _stream()), "dflash2_conv")
    return out


def dflash2_selector_walk(cand_ids, unary, projected, anchor, pred_codebook, succ_codebook, temperatures=None, uniforms=None):
    """DFlash 2's chain selector: ``(tokens [B, S] int64, probabilities [B, S, K] fp32)``."""
    assert projected.dtype in (torch.float16, torch.bfloat16) and pred_codebook.dtype == projected.dtype == succ_codebook.dtype
    b, s, k = cand_ids.shape
    dev = cand_ids.device
    c, u, z = cand_ids.to(torch.int32).contiguous(), unary.float().contiguous(), projected.contiguous()
    a, pc, qc = anchor.to(device=dev, dtype=torch.int32).contiguous(), pred_codebook.contiguous(), succ_codebook.contiguous()
    t = None if temperatures is None else temperatures.to(device=dev, dtype=torch.float32).contiguous()
    un = None if uniforms is None else uniforms.to(device=dev, dtype=torch.float32).contiguous()
    tok = torch.empty(b, s, dtype=torch.int32, device=dev)
    pr = torch.empty(b, s, k, dtype=torch.float32, device=dev)
    _check(lib().telb_dflash2_selector(_p(c), _p(u), _p(z), _p(a), _p(pc), _p(qc), _p(t), _p(un), _p(tok), _p(pr), c_int(b), c_int(s), c_int(k),
                                       c_int(z.shape[-1]), c_int(pc.shape[0]), c_int(int(z.dtype == torch.bfloat16)), _stream()),
           "dflash2_selector")
    return tok.long(), pr


def spec_accept_sampling(target_probs, tree_tokens, parents, max_path: int, uniforms):
    """Lossless tree acceptance of sampled requests on the device: ``(path [B, max_path], path_len [B], bonus [B])`` int32."""
    b, n, v = target_probs.shape
    dev = target_probs.device
    pr = target_probs.float().contiguous()
    tok, par = tree_tokens.to(device=dev, dtype=torch.int32).contiguous(), parents.to(device=dev, dtype=torch.int32).contiguous()
    u = uniforms.to(device=dev, dtype=torch.float32).contiguous()
    assert u.shape[0] == b and u.shape[1] >= max_path and u.shape[2] >= 2
    if u.shape[1] != max_path:
        u = u[:, :max_path].contiguous()
    path = torch.empty(b, max_path, dtype=torch.int32, device=dev)
    plen = torch.empty(b, dtype=torch.int32, device=dev)
    bonus = torch.empty(b, dtype=torch.int32, device=dev)
    _check(lib().telb_spec_accept_sampling(_p(pr), _p(tok), _p(par), _p(u), _p(path), _p(plen), _p(bonus), c_int(b), c_int(n), c_int(v),
                                           c_int(max_path), c_int(u.shape[2]), _stream()), "spec_accept_sampling")
    return path, plen, bonus


def markov_greedy_chain(logits, w1, w2, first_prev):
    """Greedy chain of DSpark's Markov head over ``logits [B, P, V]`` (fp32): ``P`` fused correction + arg-max launches."""
    assert w1.dtype == w2.dtype and w1.dtype in (torch.float16, torch.bfloat16) and w1.shape[1] == w2.shape[1]
    b, p, v = logits.shape
    lg, a, c = logits.float().contiguous(), w1.contiguous(), w2.contiguous()
    fp = first_prev.to(device=lg.device, dtype=torch.int32).contiguous()
    slots = torch.empty(b * p, dtype=torch.int64, device=lg.device)
    tok = torch.empty(b, p, dtype=torch.int32, device=lg.device)
    _check(lib().telb_markov_greedy_chain(_p(lg), _p(a), _p(c), _p(fp), _p(slots), _p(tok), c_int(b), c_int(p), c_int(v), c_int(a.shape[0]),
                                          c_int(a.shape[1]), c_int(int(a.dtype == torch.bfloat16)), _stream()), "markov_greedy_chain")
    return tok.long()


def lattice_chain_walk(cand_ids, transition, temperatures=None, uniforms=None):
    """Walk of a candidate lattice with per-slot ``[prev, next]`` transition scores: ``(tokens [B, S] int64, probabilities)``."""
    b, s, k = cand_ids.shape
    dev = cand_ids.device
    c, tr = cand_ids.to(torch.int32).contiguous(), transition.float().contiguous()
    t = None if temperatures is None else temperatures.to(device=dev, dtype=torch.float32).contiguous()
    un = None if uniforms is None else uniforms.to(device=dev, dtype=torch.float32).contiguous()
    tok = torch.empty(b, s, dtype=torch.int32, device=dev)
    pr = torch.empty(b, s, k, dtype=torch.float32, device=dev)
    _check(lib().telb_lattice_chain_walk(_p(c), _p(tr), _p(t), _p(un), _p(tok), _p(pr), c_int(b), c_int(s), c_int(k), _stream()),
           "lattice_chain_walk")
    return tok.long(), pr


def candidate_rescore(hidden, lm_head, cand):
    """Exact logits of each row's candidate tokens, ordered (logit descending, id ascending), with the log-softmax over the set:
    ``(ids [R, Kc] int32, log-probabilities [R, Kc] fp32)``."""
    assert hidden.dtype == lm_head.dtype and hidden.dtype in (torch.float16, torch.bfloat16)
    h, w, c = hidden.contiguous(), lm_head.contiguous(), cand.to(torch.int32).contiguous()
    rows, kc = c.shape
    ids = torch.empty(rows, kc, dtype=torch.int32, device=h.device)
    lp = torch.empty(rows, kc, dtype=torch.float32, device=h.device)
    _check(lib().telb_candidate_rescore(_p(h), _p(w), _p(c), _p(ids), _p(lp), c_int(rows), c_int(h.shape[1]), c_int(kc),
                                        c_int(w.shape[0]), c_int(int(h.dtype == torch.bfloat16)), _stream()), "candidate_rescore")
    return ids, lp


def kv_commit_path(pool, page_table, past_len, path, path_len) -> None:
    assert pool.is_contiguous() and pool.element_size() in (1, 2)
    if pool.element_size() == 1:            # FP8 pages: a row of D bytes moves as D / 2 16-bit elements
        pool = pool.view(torch.int16)
    layers, pages, _, hkv, psz, d = pool.shape
    pt, pl, pth, pln = page_table.to(torch.int32).contiguous(), past_len.to(torch.int32).contiguous(), path.contiguous(), path_len.contiguous()
    _check(lib().telb_kv_commit_path(_p(pool), _p(pt), _p(pl), _p(pth), _p(pln), c_int(path.shape[0]), c_int(path.shape[1]),
                                     c_int(page_table.shape[1]), c_int(layers), c_int(pages), c_int(hkv), c_int(psz), c_int(d),
                                     _stream()), "kv_commit_path")
