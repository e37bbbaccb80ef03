"""Linear layers: dense 16-bit, NVFP4 (W4A4 / W4A16) and INT4-AWQ, with tensor-parallel modes.

Parity: ``tensorrt_edgellm/models/linear.py`` — ``TPMode`` and Column/Row parallel classes
(:103-576), NVFP4 variants (:440-468, :765-845), INT4 (:647-757), ``make_linear`` (:1085).  The
reference lowers these to TensorRT nodes and plugins; here each ``forward`` runs the sm_100a
kernel directly (``ops.cuda``) or the PyTorch statement on CPU.

Checkpoint tensors keep their Hugging Face / ModelOpt names (``weight``, ``weight_scale``,
``weight_scale_2``, ``input_scale``, ``bias``) so loading is a plain name match; a layer that
fuses several checkpoint modules (``qkv_proj``, ``gate_up_proj``) lists them in ``sources``.
"""
from __future__ import annotations

import enum
from typing import Dict, List, Optional, Sequence

import torch
from torch import nn

from .. import ops
from ..config import (EXPANDED_QUANT_TYPES, QUANT_INT4_AWQ, QUANT_NONE, QUANT_NVFP4, QUANT_NVFP4_A16, ModelConfig)
from ..ops import reference as ref


class TPMode(enum.Enum):
    REPLICATED = "replicated"
    COL = "col"     # output features sharded; no collective
    ROW = "row"     # input features sharded; partial sums reduced by the caller's collective


def _shard(t: torch.Tensor, dim: int, rank: int, world: int) -> torch.Tensor:
    if world == 1:
        return t
    n = t.shape[dim]
    if n % world:
        raise ValueError(f"dimension {dim} of size {n} is not divisible by TP {world}")
    return t.narrow(dim, rank * (n // world), n // world).contiguous()


class LinearBase(nn.Module):
    """Common bookkeeping: logical sizes, TP placement and the checkpoint modules it fuses."""

    rs_comm = None      # set on row-parallel layers whose output may leave through a reduce-scatter epilogue

    def __init__(self, in_features: int, out_features: Sequence[int], tp_mode: TPMode, tp_size: int, tp_rank: int,
                 sources: Optional[List[str]] = None, bias: bool = False, row_ranges=None):
        super().__init__()
        self.tp_mode, self.tp_size, self.tp_rank = tp_mode, tp_size, tp_rank
        self.sources = sources
        self.full_in = in_features
        self.full_out = list(out_features)
        # row_ranges[i] = (lo, hi) overrides the even column-parallel split of segment i (replicated KV heads)
        self.row_ranges = row_ranges
        self.in_features = in_features // tp_size if tp_mode == TPMode.ROW else in_features
        self.out_sizes = [o // tp_size if tp_mode == TPMode.COL else o for o in out_features]
        if row_ranges is not None:
            self.out_sizes = [(r[1] - r[0]) if r is not None else s for r, s in zip(row_ranges, self.out_sizes)]
        self.out_features = sum(self.out_sizes)
        self.has_bias = bias

    # sharding of one source module's tensor (dim 0 = out, dim 1 = in)
    def shard_out_in(self, t: torch.Tensor, segment: int = 0) -> torch.Tensor:
        if self.tp_mode == TPMode.COL:
            if self.row_ranges is not None and self.row_ranges[segment] is not None:
                lo, hi = self.row_ranges[segment]
                return t[lo:hi].contiguous()
            return _shard(t, 0, self.tp_rank, self.tp_size)
        if self.tp_mode == TPMode.ROW and t.dim() > 1:
            return _shard(t, 1, self.tp_rank, self.tp_size)
        return t

    def load_from(self, tensors: List[Dict[str, torch.Tensor]]) -> None:
        raise NotImplementedError

    def _split_single_source(self, tensors):
        """One checkpoint module that holds several logical segments stacked along the output dim
        (e.g. a Mamba ``in_proj`` = [z | x | B | C | dt]): split it so each segment shards on its own."""
        if len(tensors) != 1 or len(self.full_out) == 1:
            return tensors
        out, off = [], 0
        for n in self.full_out:
            out.append({k: (v[off:off + n] if v.dim() >= 1 and v.shape[0] == sum(self.full_out) else v) for k, v in tensors[0].items()})
            off += n
        return out

    def finalize(self) -> None:
        """Hook run once after loading and device placement (GPU-side repacks)."""

    def fused_input_scale(self) -> Optional[torch.Tensor]:
        """Global activation scale when this layer wants its input pre-quantised by the producer
        kernel (NVFP4 W4A4 on a GPU), else None."""
        return None


class Linear(LinearBase):
    """16-bit dense linear, ``y = x Wᵀ (+ b)``."""

    def __init__(self, in_features, out_features, tp_mode=TPMode.REPLICATED, tp_size=1, tp_rank=0, sources=None,
                 bias=False, dtype=torch.bfloat16, row_ranges=None):
        super().__init__(in_features, out_features, tp_mode, tp_size, tp_rank, sources, bias, row_ranges)
        self.weight = nn.Parameter(torch.empty(self.out_features, self.in_features, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(self.out_features, dtype=dtype), requires_grad=False) if bias else None

    def load_from(self, tensors):
        tensors = self._split_single_source(tensors)
        ws = [self.shard_out_in(t["weight"], i) for i, t in enumerate(tensors)]
        self.weight.data.copy_(torch.cat(ws, dim=0).to(self.weight.dtype))
        if self.bias is not None:
            bs = []
            for i, t in enumerate(tensors):
                b = t["bias"]
                bs.append(self.shard_out_in(b, i) if self.tp_mode == TPMode.COL else b)
            b = torch.cat(bs, dim=0)
            if self.tp_mode == TPMode.ROW and self.tp_rank != 0:
                b = torch.zeros_like(b)       # the reduced sum must add the bias once
            self.bias.data.copy_(b.to(self.bias.dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda:
            if self.rs_comm is not None and self.rs_comm.use_rs(x.shape[0]):
                return self.rs_comm.gemm_reduce_scatter(self, x)        # rows go straight to their owner rank
            ag = getattr(x, "ag_wait", None)
            if ag is not None:                                          # rows still arriving from peers
                return ops.cuda_ops().gemm_fused(x, self.weight, ag, bias=self.bias)
        return ops.linear(x, self.weight, self.bias)


class NVFP4Linear(LinearBase):
    """NVFP4 weights (E2M1 pairs, E4M3 scale per 16 inputs, fp32 ``weight_scale_2``).

    ``quantize_activations`` selects W4A4 (activations quantised per 16-block with the
    calibrated ``input_scale``, block-scaled tensor-core GEMM) or W4A16.  Fused sources keep
    one global weight scale per source; it is folded into a per-output-column ``alpha``.
    """

    def __init__(self, in_features, out_features, tp_mode=TPMode.REPLICATED, tp_size=1, tp_rank=0, sources=None,
                 bias=False, dtype=torch.bfloat16, quantize_activations=True, row_ranges=None):
        super().__init__(in_features, out_features, tp_mode, tp_size, tp_rank, sources, bias, row_ranges)
        if self.in_features % 16:
            raise ValueError("NVFP4 needs in_features divisible by 16 on every rank")
        self.act_dtype = dtype
        self.quantize_activations = quantize_activations
        self.register_buffer("weight", torch.zeros(self.out_features, self.in_features // 2, dtype=torch.uint8))
        self.register_buffer("weight_scale", torch.zeros(self.out_features, self.in_features // 16, dtype=torch.float8_e4m3fn))
        self.register_buffer("weight_scale_2", torch.ones(len(self.out_sizes), dtype=torch.float32))
        self.register_buffer("input_scale", torch.ones((), dtype=torch.float32))
        self.register_buffer("alpha", torch.ones(self.out_features, dtype=torch.float32))
        self.bias = nn.Parameter(torch.zeros(self.out_features, dtype=dtype), requires_grad=False) if bias else None
        self._gpu_weight_sf = None      # scale factors repacked for the tensor-core kernel
        # gate/up projections feeding an NVFP4 down projection: on the GPU the rows are stored as blocks of 64 gate rows
        # alternating with their 64 up rows, so one 128-wide GEMM tile holds both halves of 64 SwiGLU outputs and the
        # epilogue can apply the activation and quantise (``forward_swiglu``).  Requested by the MLP, done in finalize.
        self.want_interleave = False
        self.gate_up_interleaved = False

    def _interleave_perm(self) -> torch.Tensor:
        inter = self.out_sizes[0]
        blk = torch.arange(inter, device=self.weight.device).view(inter // 64, 64)
        return torch.stack([blk, blk + inter], dim=1).reshape(-1)          # [g0..63, u0..63, g64..127, u64..127, ...]

    def load_from(self, tensors):
        self.gate_up_interleaved, self._gpu_weight_sf = False, None
        w = torch.cat([self.shard_out_in(t["weight"], i) for i, t in enumerate(tensors)], dim=0)
        sf = torch.cat([self.shard_out_in(t["weight_scale"].view(torch.uint8), i) for i, t in enumerate(tensors)], dim=0)
        self.weight.copy_(w.view(torch.uint8))
        self.weight_scale.copy_(sf.view(torch.float8_e4m3fn))
        self.weight_scale_2.copy_(torch.stack([t["weight_scale_2"].float().reshape(()) for t in tensors]))
        ins = [t["input_scale"].float().reshape(()) for t in tensors if "input_scale" in t]
        if ins:
            self.input_scale.copy_(torch.stack(ins).max())
        self._refresh_alpha()
        if self.bias is not None:
            self.bias.data.copy_(torch.cat([t["bias"] for t in tensors]).to(self.bias.dtype))

    def _refresh_alpha(self):
        per_col = torch.cat([self.weight_scale_2[i].expand(n) for i, n in enumerate(self.out_sizes)])
        gs = self.input_scale if self.quantize_activations else torch.ones_like(self.input_scale)
        self.alpha.copy_(per_col * gs)

    @torch.no_grad()
    def quantize_from(self, weights: List[torch.Tensor], input_scale: float = 1.0 / 448.0) -> None:
        """Quantise 16-bit weights (one tensor per fused source) into this layer."""
        self.gate_up_interleaved, self._gpu_weight_sf = False, None
        packs, sfs, gss = [], [], []
        for wt in weights:
            p, sf, gs = ref.nvfp4_quantize(wt.float())
            packs.append(p); sfs.append(sf.view(torch.uint8)); gss.append(gs)
        self.weight.copy_(torch.cat(packs, 0))
        self.weight_scale.copy_(torch.cat(sfs, 0).view(torch.float8_e4m3fn))
        self.weight_scale_2.copy_(torch.stack(gss))
        self.input_scale.fill_(float(input_scale))
        self._refresh_alpha()

    def dequantized_weight(self) -> torch.Tensor:
        per_row = torch.cat([self.weight_scale_2[i].expand(n) for i, n in enumerate(self.out_sizes)])
        w, sf = self.weight, self.weight_scale
        if self.gate_up_interleaved:             # back to [gate | up] row order
            inv = torch.argsort(self._interleave_perm())
            w, sf = w[inv], sf.view(torch.uint8)[inv].view(torch.float8_e4m3fn)
        return ref.nvfp4_dequantize(w, sf, torch.ones((), device=self.weight.device)) * per_row[:, None]

    @torch.no_grad()
    def finalize(self):
        if self.weight.is_cuda:
            if (self.want_interleave and not self.gate_up_interleaved and self.bias is None and len(self.out_sizes) == 2
                    and self.out_sizes[0] == self.out_sizes[1] and self.out_sizes[0] % 64 == 0):
                perm = self._interleave_perm()
                self.weight.copy_(self.weight[perm])
                self.weight_scale.copy_(self.weight_scale.view(torch.uint8)[perm].view(torch.float8_e4m3fn))
                self.alpha.copy_(self.alpha[perm])
                self.gate_up_interleaved = True
            self._gpu_weight_sf = ops.cuda_ops().nvfp4_swizzle_scales(self.weight_scale)

    SWIGLU_SMALL_MAX = 64        # rows up to which the decode-size kernel carries the SwiGLU epilogue

    def forward_swiglu(self, x, out_scale: torch.Tensor):
        """``quantise(silu(gate) * up)`` of this (interleaved) gate/up projection for NVFP4 input rows ``x``: more than 128
        rows in the prefill kernel's epilogue, up to 64 rows in the decode-size kernel's."""
        cu = ops.cuda_ops()
        if x.shape[0] <= self.SWIGLU_SMALL_MAX:
            return cu.gemm_skinny_swiglu(x, self.weight, self._gpu_weight_sf, self.alpha, out_scale, getattr(x, "ag_wait", None))
        return cu.gemm_nvfp4_swiglu(x, self.weight, self._gpu_weight_sf, self.alpha, out_scale, getattr(x, "ag_wait", None))

    def fused_input_scale(self):
        return self.input_scale if (self.quantize_activations and self.weight.is_cuda) else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda:
            if self._gpu_weight_sf is None:
                self.finalize()
            if self.quantize_activations:
                if self.rs_comm is not None and self.rs_comm.use_rs(x.shape[0]):
                    return self.rs_comm.gemm_reduce_scatter(self, x)
                ag = getattr(x, "ag_wait", None)
                if ag is not None:
                    return ops.cuda_ops().gemm_fused(x, self.weight, ag, w_sf=self._gpu_weight_sf, alpha=self.alpha, bias=self.bias)
            return ops.cuda_ops().nvfp4_linear(x, self.weight, self._gpu_weight_sf, self.alpha, self.input_scale,
                                               self.bias, self.quantize_activations)
        xa = x.float()
        if self.quantize_activations:
            xa = ref.nvfp4_act_qdq(xa, self.input_scale)
        y = xa @ self.dequantized_weight().t()
        if self.bias is not None:
            y = y + self.bias.float()
        return y.to(x.dtype)


class Int4AwqLinear(LinearBase):
    """INT4 group-wise weights in the ModelOpt prepacked layout (``weight [out/2, in]`` uint8,
    ``weight_scale [out, in/g]``, optional ``pre_quant_scale [in]``)."""

    def __init__(self, in_features, out_features, tp_mode=TPMode.REPLICATED, tp_size=1, tp_rank=0, sources=None,
                 bias=False, dtype=torch.bfloat16, group_size=128, row_ranges=None):
        super().__init__(in_features, out_features, tp_mode, tp_size, tp_rank, sources, bias, row_ranges)
        self.group = group_size
        self.register_buffer("weight", torch.zeros(self.out_features // 2, self.in_features, dtype=torch.uint8))
        self.register_buffer("weight_scale", torch.ones(self.out_features, self.in_features // group_size, dtype=dtype))
        self.register_buffer("pre_quant_scale", torch.ones(self.in_features, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(self.out_features, dtype=dtype), requires_grad=False) if bias else None
        self._dense = None
        self._pqs_is_one = None          # pre_quant_scale of all ones (a checkpoint without AWQ smoothing): skip the multiply

    def load_from(self, tensors):
        self._pqs_is_one = None
        self.weight.copy_(torch.cat([self.shard_out_in(t["weight"].view(torch.uint8)) for t in tensors], 0))
        self.weight_scale.copy_(torch.cat([self.shard_out_in(t["weight_scale"]) for t in tensors], 0).to(self.weight_scale.dtype))
        if "pre_quant_scale" in tensors[0]:
            pq = tensors[0]["pre_quant_scale"]
            if self.tp_mode == TPMode.ROW:
                pq = _shard(pq, 0, self.tp_rank, self.tp_size)
            self.pre_quant_scale.copy_(pq.to(self.pre_quant_scale.dtype))

    @torch.no_grad()
    def quantize_from(self, weights: List[torch.Tensor]) -> None:
        w = torch.cat([wt.float() for wt in weights], 0)
        g = self.group
        wg = w.reshape(w.shape[0], w.shape[1] // g, g)
        scale = (wg.abs().amax(-1) / 7.0).clamp(min=1e-8)
        q = (torch.round(wg / scale[..., None]).clamp(-8, 7) + 8).to(torch.uint8).reshape(w.shape)
        self.weight.copy_(q[0::2] | (q[1::2] << 4))
        self.weight_scale.copy_(scale.to(self.weight_scale.dtype))
        self._dense = None

    def dequantized_weight(self) -> torch.Tensor:
        return ref.int4_awq_dequantize(self.weight, self.weight_scale, None, self.group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._pqs_is_one is None:
            self._pqs_is_one = bool((self.pre_quant_scale == 1).all())
        xs = x if self._pqs_is_one else (x.float() * self.pre_quant_scale.float()).to(x.dtype)
        if x.is_cuda:
            # W4A16 with the weights kept in 4 bits: decode-size steps expand the codes tile by tile inside the GEMM
            # kernel (only 4-bit weights cross HBM); prefill-size steps expand into a temporary and run the dense GEMM
            return ops.cuda_ops().gemm_int4_awq(xs, self.weight, self.weight_scale, self.group, bias=self.bias)
        y = xs.float() @ self.dequantized_weight().t()
        if self.bias is not None:
            y = y + self.bias.float()
        return y.to(x.dtype)


class ExpandedLinear(Linear):
    """A linear whose checkpoint stores a weight-only format (GPTQ, AutoAWQ, FP8, INT8-SQ, MXFP8, Q8_0): the tensors
    are decoded to a dense matrix once while loading and the layer then runs as a 16-bit :class:`Linear`.

    Parity: the weight-only members of ``tensorrt_edgellm/models/linear.py:647-920`` and their plugins
    (``int4GroupwiseGemmPlugin``, ``q8_0LinearPlugin`` …); here the tcgen05 16-bit GEMM serves all of them."""

    def __init__(self, in_features, out_features, quant_type: str, zero_point_offset: int = 1, **kw):
        super().__init__(in_features, out_features, **kw)
        self.quant_type, self.zero_point_offset = quant_type, zero_point_offset

    def load_from(self, tensors):
        from ..checkpoint.repacking import decode_bundle
        dense = []
        for t in tensors:
            w = decode_bundle(t, self.quant_type, self.zero_point_offset)
            b = {"weight": w if w is not None else t["weight"]}
            if "bias" in t:
                b["bias"] = t["bias"]
            dense.append(b)
        super().load_from(dense)


def make_linear(cfg: ModelConfig, name: str, in_features: int, out_features: Sequence[int],
                tp_mode: TPMode = TPMode.REPLICATED, sources: Optional[List[str]] = None, bias: bool = False,
                quantizable: bool = True, row_ranges=None) -> LinearBase:
    """Build the linear layer the checkpoint's quantisation calls for.  ``name`` is the fully
    qualified module name used for exclusion matching (``lm_head`` stays 16-bit unless the
    checkpoint says otherwise)."""
    tp_size, tp_rank = (cfg.tp_size, cfg.tp_rank) if tp_mode != TPMode.REPLICATED else (1, 0)
    qt = cfg.quant.module_quant_type(name) if quantizable else QUANT_NONE
    if name.endswith("lm_head"):
        qt = cfg.quant.lm_head_quant_type
    kw = dict(tp_mode=tp_mode, tp_size=tp_size, tp_rank=tp_rank, sources=sources, bias=bias, dtype=cfg.compute_dtype)
    if row_ranges is not None:
        kw["row_ranges"] = row_ranges
    if qt in (QUANT_NVFP4, QUANT_NVFP4_A16):
        return NVFP4Linear(in_features, out_features, quantize_activations=(qt == QUANT_NVFP4 and cfg.quant.quantize_activations), **kw)
    if qt == QUANT_INT4_AWQ:
        if cfg.quant.awq_layout == "autoawq":
            return ExpandedLinear(in_features, out_features, quant_type=qt, **kw)
        return Int4AwqLinear(in_features, out_features, group_size=cfg.quant.group_size or 128, **kw)
    if qt in EXPANDED_QUANT_TYPES:
        return ExpandedLinear(in_features, out_features, quant_type=qt, zero_point_offset=cfg.quant.gptq_zero_point_offset, **kw)
    return Linear(in_features, out_features, **kw)
