"""Dense Llama / Qwen-style decoder (pre-norm, GQA, SwiGLU) on the ragged step ABI.

Parity: ``tensorrt_edgellm/models/default/modeling_default.py`` — ``RMSNorm`` :163-182,
``Attention`` :190-461 (q/k/v column-parallel, o row-parallel, qk-norm before RoPE),
``fuse_qkv_projections`` :523, ``MLP`` :696-735, ``DecoderLayer`` :743-805, ``Transformer``
:813-973, ``CausalLM`` :985.  The reference module is an export graph whose attention body
returns zeros; this one executes: every leaf is an ``ops`` call.

Each row-parallel output (o_proj, down_proj) flows straight into a residual-add + RMSNorm.
That pair is the seam where tensor parallelism reduces partial sums, so the layer calls
``comm.add_rmsnorm`` and the communicator decides between a local kernel (TP=1), NCCL
all-reduce followed by the kernel (baseline) and the fused peer-memory kernel.
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..ops.meta import StepMeta
from ..parallel.comm import LocalComm
from .linear import NVFP4Linear, TPMode, make_linear


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype=torch.bfloat16):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        tp = cfg.tp_size
        self.layer_idx = layer_idx
        self.head_dim = cfg.head_dim
        self.num_q_heads = cfg.num_attention_heads // tp
        self.num_kv_heads = max(cfg.num_key_value_heads // tp, 1)
        kv_ranges = None
        if cfg.num_key_value_heads % tp:
            # fewer KV heads than ranks: each KV head is replicated on tp / Hkv consecutive ranks
            if tp % cfg.num_key_value_heads:
                raise ValueError("the TP degree must be a multiple or a divisor of the KV head count")
            kvh = cfg.tp_rank // (tp // cfg.num_key_value_heads)
            kv_ranges = [None, (kvh * cfg.head_dim, (kvh + 1) * cfg.head_dim), (kvh * cfg.head_dim, (kvh + 1) * cfg.head_dim)]
        self.scale = cfg.head_dim ** -0.5
        self.sliding_window = cfg.sliding_window
        self.eps = cfg.rms_norm_eps
        h = cfg.hidden_size
        # a KV-shared layer attends over its donor's cache (the decoder stack hands it that layer) and projects queries only
        self.kv_donor = cfg.kv_donor(layer_idx) if hasattr(cfg, "kv_donor") else -1
        win = cfg.layer_windows[layer_idx] if cfg.layer_windows else (cfg.sliding_window or 0)
        self.k_eq_v = bool(getattr(cfg, "attention_k_eq_v", False)) and not win       # full-attention layers only
        self.value_norm = bool(getattr(cfg, "has_value_norm", False))
        if self.kv_donor >= 0:
            self.qkv_proj = make_linear(cfg, f"{prefix}.qkv_proj", h, [cfg.q_size], TPMode.COL, sources=["q_proj"], bias=cfg.attention_bias)
        elif self.k_eq_v:
            if kv_ranges is not None:
                raise ValueError("attention_k_eq_v with replicated KV heads under tensor parallelism is not built")
            self.qkv_proj = make_linear(cfg, f"{prefix}.qkv_proj", h, [cfg.q_size, cfg.kv_size], TPMode.COL, sources=["q_proj", "k_proj"],
                                        bias=cfg.attention_bias)
        else:
            self.qkv_proj = make_linear(cfg, f"{prefix}.qkv_proj", h, [cfg.q_size, cfg.kv_size, cfg.kv_size], TPMode.COL,
                                        sources=["q_proj", "k_proj", "v_proj"], bias=cfg.attention_bias, row_ranges=kv_ranges)
        self.o_proj = make_linear(cfg, f"{prefix}.o_proj", cfg.q_size, [h], TPMode.ROW)
        if cfg.has_qk_norm:
            self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, cfg.compute_dtype)
            self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, cfg.compute_dtype)
        else:
            self.q_norm = self.k_norm = None
        self.prefix = prefix
        self.register_buffer("kv_scales", torch.ones(2, dtype=torch.float32))      # FP8 KV cache: K and V dequantisation scales
        if getattr(cfg, "attention_sink_bias", False):
            # one learned logit per (local) query head with no value row: it only grows the softmax denominator
            # (reference: tensorrt_edgellm/config.py:691-692, the draft models' attention_sink_bias buffer)
            self.register_buffer("attention_sink_bias", torch.zeros(self.num_q_heads, dtype=torch.float32))
        else:
            self.attention_sink_bias = None

    def _forward_fp8_decode(self, qkv, meta, pool_layer, cos_sin):
        """Decode-shaped step over FP8 pages: the new rows pass through the staging layer only to be quantised into the pool
        (no page is expanded), the queries are cast to E4M3 in the same launch, and the decode kernel reads the pool in place."""
        cu = ops.cuda_ops()
        stage = cu.kv_fp8_stage(pool_layer, qkv.dtype)
        q = ops.rope_kv_write(qkv, stage, meta, cos_sin, self.num_q_heads, self.num_kv_heads, self.head_dim,
                              None if self.q_norm is None else self.q_norm.weight,
                              None if self.k_norm is None else self.k_norm.weight, self.eps)
        q8 = cu.kv_fp8_store(pool_layer, stage, meta, self.kv_scales, q)
        gs = self.o_proj.fused_input_scale() if hasattr(self.o_proj, "fused_input_scale") else None
        o = cu.paged_attention_decode_fp8(q8, pool_layer, meta, self.scale, self.sliding_window, self.kv_scales, qkv.dtype,
                                          out_scale=gs, sinks=self.attention_sink_bias)
        return self.o_proj(o if gs is not None else o.reshape(o.shape[0], -1))

    def load_checkpoint(self, fetch) -> bool:
        """FP8 KV-cache scales of quantised checkpoints (``k_proj.k_scale`` / ``v_proj.v_scale``, one per layer)."""
        for i, name in enumerate(("k_proj.k_scale", "v_proj.v_scale")):
            t = fetch(f"{self.prefix}.{name}")
            if t is not None:
                self.kv_scales[i] = t.float().reshape(-1)[0]
        return False

    def _derive_values(self, qkv: torch.Tensor) -> torch.Tensor:
        """Packed ``[q | k | v]`` of the variants whose values are not a plain projection: ``v = k`` (raw, before the key norm and
        RoPE) when the layer has no value projection, and a weightless per-head RMSNorm on ``v``."""
        qn, kn = self.num_q_heads * self.head_dim, self.num_kv_heads * self.head_dim
        q, k = qkv[:, :qn], qkv[:, qn:qn + kn]
        v = k if self.k_eq_v else qkv[:, qn + kn:]
        if self.value_norm:
            vf = v.float().reshape(-1, self.num_kv_heads, self.head_dim)
            v = (vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + self.eps)).reshape(v.shape[0], kn).to(qkv.dtype)
        return torch.cat((q, k, v), dim=-1)

    def _forward_shared_kv(self, x, meta, kv_layer, cos_sin):
        """KV-shared layer: queries only; ``kv_layer`` is the donor's cache, already holding this step's rows."""
        if kv_layer.dtype == torch.float8_e4m3fn:
            raise NotImplementedError("KV-shared layers over an FP8 cache are not built")
        q = ops.rope_q(self.qkv_proj(x), kv_layer, meta, cos_sin, self.num_q_heads, self.head_dim,
                       None if self.q_norm is None else self.q_norm.weight, self.eps)
        o = ops.paged_attention(q, kv_layer, meta, self.scale, self.sliding_window, self.attention_sink_bias)
        return self.o_proj(o.reshape(o.shape[0], -1))

    def forward(self, x: torch.Tensor, meta: StepMeta, kv_layer: torch.Tensor, cos_sin: torch.Tensor) -> torch.Tensor:
        if self.kv_donor >= 0:
            return self._forward_shared_kv(x, meta, kv_layer, cos_sin)
        qkv = self.qkv_proj(x)
        if self.k_eq_v or self.value_norm:
            qkv = self._derive_values(qkv)
        pool_layer = None
        if kv_layer.dtype == torch.float8_e4m3fn:
            pool_layer = kv_layer
            if qkv.is_cuda and ops.cuda_ops().fp8_decode_ok((qkv.shape[0], self.num_q_heads, self.head_dim), kv_layer.shape[2], meta):
                return self._forward_fp8_decode(qkv, meta, pool_layer, cos_sin)
            # FP8 pages, prefill-size step: attention works on the 16-bit staging copy of the pages this step touches; the new
            # rows are quantised into the pool (and rounded in the copy) right after they are written
            kv_layer = ops.kv_fp8_prepare(pool_layer, meta, self.kv_scales, qkv.dtype, self.sliding_window or 0)
        q = ops.rope_kv_write(qkv, kv_layer, meta, cos_sin, self.num_q_heads, self.num_kv_heads, self.head_dim,
                              None if self.q_norm is None else self.q_norm.weight,
                              None if self.k_norm is None else self.k_norm.weight, self.eps)
        if pool_layer is not None:
            ops.kv_fp8_commit(pool_layer, kv_layer, meta, self.kv_scales)
        gs = self.o_proj.fused_input_scale() if hasattr(self.o_proj, "fused_input_scale") else None
        sinks = self.attention_sink_bias
        if gs is not None and q.is_cuda and ops.cuda_ops().decode_attention_quant_ok(q.shape, kv_layer.shape[2], meta):
            # decode step into an NVFP4 projection: the attention epilogue quantises for it
            return self.o_proj(ops.cuda_ops().paged_attention_quant(q, kv_layer, meta, self.scale, self.sliding_window, gs, sinks=sinks))
        o = ops.paged_attention(q, kv_layer, meta, self.scale, self.sliding_window, sinks)
        return self.o_proj(o.reshape(o.shape[0], -1))


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str, intermediate: Optional[int] = None):
        super().__init__()
        inter = intermediate or cfg.intermediate_size
        self.act = cfg.hidden_act
        if self.act in ("silu", "swiglu"):
            self.gate_up_proj = make_linear(cfg, f"{prefix}.gate_up_proj", cfg.hidden_size, [inter, inter], TPMode.COL,
                                            sources=["gate_proj", "up_proj"])
        else:   # non-gated (relu²) MLP
            self.gate_up_proj = make_linear(cfg, f"{prefix}.up_proj", cfg.hidden_size, [inter], TPMode.COL,
                                            sources=["up_proj"])
        self.down_proj = make_linear(cfg, f"{prefix}.down_proj", inter, [cfg.hidden_size], TPMode.ROW)
        # NVFP4 W4A4 on both projections: SwiGLU and the quantisation of the down projection's input move into the
        # gate/up GEMM's epilogue at prefill sizes (TELB_DISABLE_SWIGLU_FUSION=1 keeps the separate kernel)
        if (self.act in ("silu", "swiglu") and isinstance(self.gate_up_proj, NVFP4Linear) and isinstance(self.down_proj, NVFP4Linear)
                and self.gate_up_proj.quantize_activations and self.down_proj.quantize_activations
                and os.environ.get("TELB_DISABLE_SWIGLU_FUSION", "0") != "1"):
            self.gate_up_proj.want_interleave = True

    def forward(self, x):
        gp = self.gate_up_proj
        if getattr(gp, "want_interleave", False) and getattr(x, "is_cuda", False):
            if gp._gpu_weight_sf is None:
                gp.finalize()
            if gp.gate_up_interleaved:
                scale = self.down_proj.fused_input_scale()
                rows = x.shape[0]
                # NVFP4 rows in: prefill sizes fuse in the wide kernel's epilogue, decode sizes in the skinny kernel's
                small = (rows <= gp.SWIGLU_SMALL_MAX and gp.bias is None
                         and os.environ.get("TELB_DISABLE_SWIGLU_DECODE_FUSION", "0") != "1")
                if not isinstance(x, torch.Tensor) and (rows > 128 or small):
                    return self.down_proj(gp.forward_swiglu(x, scale))
                return self.down_proj(ops.swiglu(gp(x), scale, interleaved=True))
        gu = gp(x)
        a = ops.swiglu(gu, self.down_proj.fused_input_scale()) if self.act in ("silu", "swiglu") else ops.relu2(gu)
        return self.down_proj(a)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int):
        super().__init__()
        p = f"model.layers.{layer_idx}"
        self.self_attn = Attention(cfg, layer_idx, f"{p}.self_attn")
        self.mlp = MLP(cfg, f"{p}.mlp")
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)

    def forward(self, h, residual, meta, kv_layer, cos_sin, comm):
        qs_attn = self.self_attn.qkv_proj.fused_input_scale()
        if residual is None:
            residual = h
            x = ops.rmsnorm_maybe_quant(h, self.input_layernorm.weight, self.input_layernorm.eps, qs_attn)
        else:
            x, residual = comm.add_rmsnorm(h, residual, self.input_layernorm.weight, self.input_layernorm.eps, qs_attn,
                                           defer_gather=True)
        a = self.self_attn(x, meta, kv_layer, cos_sin)
        # the normalised rows feed one GEMM each (QKV above, gate/up below), which may wait for the gather itself
        x, residual = comm.add_rmsnorm(a, residual, self.post_attention_layernorm.weight,
                                       self.post_attention_layernorm.eps, self.mlp.gate_up_proj.fused_input_scale(),
                                       defer_gather=True)
        return self.mlp(x), residual


class Transformer(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=cfg.compute_dtype)
        self.embed_tokens.weight.requires_grad_(False)
        self.layers = nn.ModuleList([DecoderLayer(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)

    def forward(self, ids, meta, kv_cache, cos_sin, comm, inputs_embeds=None, capture_layers=()):
        h = ops.embedding(ids, self.embed_tokens.weight) if inputs_embeds is None else inputs_embeds
        residual = None
        taps = []
        rs_was = getattr(comm, "rs_enabled", None)
        if capture_layers and rs_was:
            comm.rs_enabled = False          # tapping hidden states needs the whole residual stream on every rank
        for i, layer in enumerate(self.layers):
            donor = getattr(getattr(layer, "self_attn", None), "kv_donor", -1)
            h, residual = layer(h, residual, meta, kv_cache[donor if donor >= 0 else i], cos_sin, comm)
            if meta.deepstack is not None and i in meta.deepstack:
                # deepstack binding (``cpp/runtime/features/deepstackBinding.cpp`` in the reference): the hidden state of a
                # row is h + residual here, so adding the level's features to h adds them to the stream
                rows, feats = meta.deepstack[i]
                h = h.index_add(0, rows.to(h.device), (feats.to(h.device, h.dtype) / comm.world_size) if comm.world_size > 1
                                else feats.to(h.device, h.dtype))
            if i in capture_layers:
                taps.append((h.float() + residual.float()).to(h.dtype) if comm.world_size == 1
                            else comm.all_reduce(h).add_(residual))
        x, _ = comm.add_rmsnorm(h, residual, self.norm.weight, self.norm.eps)
        if capture_layers and rs_was:
            comm.rs_enabled = True
        return (x, taps) if capture_layers else x


class CausalLM(nn.Module):
    """Decoder + LM head.  ``forward`` returns logits only for ``meta.logits_idx`` rows."""

    # checkpoint module name → (fused layer attribute, ordered source names)
    packed_modules = {"qkv_proj": ["q_proj", "k_proj", "v_proj"], "gate_up_proj": ["gate_proj", "up_proj"]}

    transformer_cls = None      # subclasses substitute their own decoder stack

    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__()
        self.cfg = cfg
        self.comm = comm or LocalComm()
        self.model = (self.transformer_cls or Transformer)(cfg)
        # The LM head is vocabulary-sharded under TP; the sampler merges per-shard candidates.
        self.lm_head = make_linear(cfg, "lm_head", cfg.hidden_size, [cfg.vocab_size],
                                   TPMode.COL if cfg.tp_size > 1 and cfg.vocab_size % cfg.tp_size == 0 else TPMode.REPLICATED)
        self._cos_sin: Optional[torch.Tensor] = None
        if self.transformer_cls is None and hasattr(self.comm, "gemm_reduce_scatter"):
            # dense decoder: every row-parallel projection is followed by comm.add_rmsnorm, so its GEMM may
            # hand the rows to their owner ranks itself (reduce-scatter epilogue) at prefill sizes
            for layer in self.model.layers:
                layer.self_attn.o_proj.rs_comm = self.comm
                layer.mlp.down_proj.rs_comm = self.comm

    def cos_sin(self, device) -> torch.Tensor:
        if self._cos_sin is None or self._cos_sin.device != torch.device(device):
            self._cos_sin = ops.rope_cos_sin(self.cfg.max_position_embeddings, self.cfg.rotary_dim,
                                                 self.cfg.rope_theta, self.cfg.rope_scaling, device=device)
        return self._cos_sin

    def hidden_states(self, ids, meta, kv_cache, inputs_embeds=None, capture_layers=()):
        dev = ids.device if inputs_embeds is None else inputs_embeds.device
        cs = self.cos_sin(dev)
        if meta.positions3 is not None and self.cfg.mrope_section and meta.rope_rows is None:
            # multimodal RoPE: one [T, D] cos / sin row per token, built from its (t, h, w) position, shared by all layers
            meta.rope_rows = ops.mrope_rows(cs, meta.positions3, self.cfg.mrope_section)
            meta.rope_pos = torch.arange(meta.num_tokens, dtype=torch.int32, device=dev)
        return self.model(ids, meta, kv_cache, cs, self.comm, inputs_embeds, capture_layers)

    def logits_from_hidden(self, x: torch.Tensor, meta: StepMeta) -> torch.Tensor:
        rows = x if meta.logits_idx.numel() == x.shape[0] else x.index_select(0, meta.logits_idx.long())
        logits = self.lm_head(rows)
        if self.lm_head.tp_mode == TPMode.COL and self.comm.world_size > 1:
            logits = self.comm.all_gather_cols(logits)
        return logits

    def forward(self, ids: torch.Tensor, meta: StepMeta, kv_cache: torch.Tensor,
                inputs_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.hidden_states(ids, meta, kv_cache, inputs_embeds)
        return self.logits_from_hidden(x, meta)

    def greedy_tokens(self, ids: torch.Tensor, meta: StepMeta, kv_cache: torch.Tensor) -> torch.Tensor:
        """Greedy next token of every ``meta.logits_idx`` row (int32 ids of the model's vocabulary).

        With a vocabulary-sharded head each rank reduces its own shard to one (value, id) candidate per row and only
        those candidates cross the link (``comm.argmax_sharded``): ``world x rows x 8`` bytes instead of the
        ``rows x vocab`` logits of a full gather.  The result equals ``argmax`` of the gathered logits, ties included."""
        return self.greedy_from_hidden(self.hidden_states(ids, meta, kv_cache), meta)

    def greedy_from_hidden(self, x: torch.Tensor, meta: StepMeta) -> torch.Tensor:
        """The greedy pick of :meth:`greedy_tokens` for final hidden states that the caller already holds (speculative
        verification keeps the tapped layers of the same pass)."""
        sharded = (self.lm_head.tp_mode == TPMode.COL and self.comm.world_size > 1 and hasattr(self.comm, "argmax_sharded")
                   and type(self).logits_from_hidden is CausalLM.logits_from_hidden)
        if not sharded:
            return ops.argmax(self.logits_from_hidden(x, meta))
        rows = x if meta.logits_idx.numel() == x.shape[0] else x.index_select(0, meta.logits_idx.long())
        return self.comm.argmax_sharded(self.lm_head(rows))

    def candidates_from_hidden(self, x: torch.Tensor, meta: StepMeta, k: int):
        """The sampler's candidate set without the full logits: every rank takes the ``k`` best logits of its vocabulary shard
        and the ranks exchange those (``2 k`` numbers per row and rank instead of ``V / world`` logits).  The ``k`` best of
        the whole vocabulary are always among them, so top-k / top-p sampling over the candidates equals sampling over the
        gathered logits.  Returns ``(values [B, world · k] fp32, token ids [B, world · k] int64)``; with one rank (or a
        replicated head) simply the top ``k``."""
        rows = x if meta.logits_idx.numel() == x.shape[0] else x.index_select(0, meta.logits_idx.long())
        shard = self.lm_head(rows).float()
        kk = min(int(k), shard.shape[-1])
        vals, idx = shard.topk(kk, dim=-1)
        if not (self.lm_head.tp_mode == TPMode.COL and self.comm.world_size > 1):
            return vals, idx
        if self.cfg.vocab_size >= 1 << 24:
            raise ValueError("candidate exchange packs token ids into fp32: the vocabulary must be below 2^24")
        idx = idx + self.comm.rank * shard.shape[-1]
        w, b = self.comm.world_size, vals.shape[0]
        g = self.comm.all_gather_cols(torch.cat([vals, idx.to(torch.float32)], dim=-1).contiguous()).view(b, w, 2, kk)
        return g[:, :, 0].reshape(b, w * kk).contiguous(), g[:, :, 1].reshape(b, w * kk).long()

    def supports_candidate_sampling(self) -> bool:
        """Whether :meth:`candidates_from_hidden` describes this model's logits (no transform between head and sampler)."""
        return type(self).logits_from_hidden is CausalLM.logits_from_hidden

    def finalize(self):
        for m in self.modules():
            if hasattr(m, "finalize") and m is not self:
                m.finalize()
        return self
