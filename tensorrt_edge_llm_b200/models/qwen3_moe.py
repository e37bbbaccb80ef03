"""Qwen3-MoE style decoder: dense attention + sparse mixture-of-experts MLP.

Parity: ``tensorrt_edgellm/models/qwen3_moe/modeling_qwen3_moe.py`` — router ``mlp.gate.weight
[E,H]`` (:116-127), per-expert gate/up/down (:135-203), softmax top-k with renormalisation,
NVFP4 expert repack (:809-883) and the plugin dispatch (:954-1070).  Here the expert path is:
route → align (128-row padded expert segments) → gather (+NVFP4 quantise) → grouped FC1 →
SwiGLU (+quantise) → grouped FC2 → weighted combine, every step a kernel of this package.

Parallelism.  Attention is tensor-parallel as in the dense model.  Experts are either
intermediate-sharded (TP-MoE, ``ep_size == 1``) or expert-sharded (EP, ``ep_size > 1``): each
rank owns ``E / ep`` experts and, because the attention output is already replicated on every
rank, needs no dispatch transfer — it simply skips tokens routed elsewhere.  Either way the
block returns a partial sum that the next ``comm.add_rmsnorm`` reduces (the combine all-reduce
fused with residual add + norm).
"""
from __future__ import annotations

from typing import Optional

import os

import torch
from torch import nn

from .. import ops
from ..config import QUANT_NVFP4, ModelConfig
from ..model import register_model
from ..ops import reference as ref
from .default import Attention, CausalLM, RMSNorm, Transformer
from .linear import Linear, TPMode


class MoEBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        self.cfg = cfg
        self.prefix = prefix
        self.top_k = cfg.num_experts_per_tok
        self.num_experts = cfg.num_experts
        ep, tp = cfg.mapping.ep_size, cfg.mapping.tp_size
        self.ep_size, self.ep_rank = ep, cfg.mapping.ep_rank
        if ep > 1:
            if cfg.num_experts % ep:
                raise ValueError("experts must divide evenly over the expert-parallel ranks")
            self.e_lo = self.ep_rank * (cfg.num_experts // ep)
            self.e_hi = self.e_lo + cfg.num_experts // ep
            self.inter = cfg.moe_intermediate_size
            self.i_lo = 0
        else:
            self.e_lo, self.e_hi = 0, cfg.num_experts
            if cfg.moe_intermediate_size % tp:
                raise ValueError("expert intermediate size must divide over the TP ranks")
            self.inter = cfg.moe_intermediate_size // tp
            self.i_lo = cfg.tp_rank * self.inter
        self.e_local = self.e_hi - self.e_lo
        h, i, dt = cfg.hidden_size, self.inter, cfg.compute_dtype
        self.nvfp4 = cfg.quant.module_quant_type(f"{prefix}.experts") == QUANT_NVFP4
        self.gate = Linear(h, [cfg.num_experts], dtype=dt)
        # Shared expert (Qwen2-MoE / Qwen3-Next style, ``modeling_qwen3_moe.py:331-333`` in the reference): a dense SwiGLU MLP
        # every token passes through, scaled per token by sigmoid(shared_expert_gate · x) and added to the routed sum.
        # It is tensor-parallel like a dense MLP, so its partial sum reduces with the routed experts' in the next add + norm.
        self.shared_expert = None
        self.shared_expert_gate = None
        if getattr(cfg, "shared_expert_intermediate_size", 0) > 0:
            from .default import MLP
            self.shared_expert = MLP(cfg, f"{prefix}.shared_expert", intermediate=cfg.shared_expert_intermediate_size)
            self.shared_expert_gate = Linear(h, [1], dtype=dt)
            self._gate8 = None              # the [1, H] gate padded to eight rows for the tensor-core GEMM
        if self.nvfp4:
            self.register_buffer("w13", torch.zeros(self.e_local * 2 * i, h // 2, dtype=torch.uint8))
            self.register_buffer("w13_scale", torch.zeros(self.e_local * 2 * i, h // 16, dtype=torch.float8_e4m3fn))
            self.register_buffer("w13_alpha", torch.ones(self.e_local * 2 * i, dtype=torch.float32))     # scale_2 x input scale
            self.register_buffer("w2", torch.zeros(self.e_local * h, i // 2, dtype=torch.uint8))
            self.register_buffer("w2_scale", torch.zeros(self.e_local * h, i // 16, dtype=torch.float8_e4m3fn))
            self.register_buffer("w2_alpha", torch.ones(self.e_local * h, dtype=torch.float32))
            self.register_buffer("w13_scale_2", torch.ones(self.e_local, 2, dtype=torch.float32))
            self.register_buffer("w2_scale_2", torch.ones(self.e_local, dtype=torch.float32))
            self.register_buffer("input_scale", torch.tensor(1.0 / 448.0))
            self.register_buffer("down_input_scale", torch.tensor(1.0 / 448.0))
            self._w13_sf = self._w2_sf = None
        else:
            self.w13 = nn.Parameter(torch.empty(self.e_local * 2 * i, h, dtype=dt), requires_grad=False)
            self.w2 = nn.Parameter(torch.empty(self.e_local * h, i, dtype=dt), requires_grad=False)

    # ---- loading ---------------------------------------------------------------------------------
    @torch.no_grad()
    def load_checkpoint(self, fetch) -> bool:
        """Fill the stacked expert tensors from per-expert checkpoint modules.  ``fetch(name)`` returns
        a tensor or None.  Returns False when the checkpoint holds no experts for this block."""
        i, h = self.inter, self.cfg.hidden_size
        found = False
        for le, e in enumerate(range(self.e_lo, self.e_hi)):
            base = f"{self.prefix}.experts.{e}"
            g, u, d = (fetch(f"{base}.{n}.weight") for n in ("gate_proj", "up_proj", "down_proj"))
            if g is None:
                continue
            found = True
            if self.nvfp4:
                rows = slice(self.i_lo, self.i_lo + i)
                gs, us, ds = (fetch(f"{base}.{n}.weight_scale").view(torch.uint8) for n in ("gate_proj", "up_proj", "down_proj"))
                self.w13[le * 2 * i: le * 2 * i + i] = g.view(torch.uint8)[rows]
                self.w13[le * 2 * i + i: (le + 1) * 2 * i] = u.view(torch.uint8)[rows]
                self.w13_scale.view(torch.uint8)[le * 2 * i: le * 2 * i + i] = gs[rows]
                self.w13_scale.view(torch.uint8)[le * 2 * i + i: (le + 1) * 2 * i] = us[rows]
                self.w2[le * h:(le + 1) * h] = d.view(torch.uint8)[:, self.i_lo // 2:(self.i_lo + i) // 2]
                self.w2_scale.view(torch.uint8)[le * h:(le + 1) * h] = ds[:, self.i_lo // 16:(self.i_lo + i) // 16]
                self.w13_scale_2[le, 0] = fetch(f"{base}.gate_proj.weight_scale_2").float().reshape(())
                self.w13_scale_2[le, 1] = fetch(f"{base}.up_proj.weight_scale_2").float().reshape(())
                self.w2_scale_2[le] = fetch(f"{base}.down_proj.weight_scale_2").float().reshape(())
                ins = fetch(f"{base}.gate_proj.input_scale")
                if ins is not None:
                    self.input_scale.copy_(torch.maximum(self.input_scale if le else ins.float().reshape(()), ins.float().reshape(())))
                dins = fetch(f"{base}.down_proj.input_scale")
                if dins is not None:
                    self.down_input_scale.copy_(torch.maximum(self.down_input_scale if le else dins.float().reshape(()), dins.float().reshape(())))
            else:
                dt = self.w13.dtype
                self.w13.data[le * 2 * i: le * 2 * i + i] = g[self.i_lo:self.i_lo + i].to(dt)
                self.w13.data[le * 2 * i + i:(le + 1) * 2 * i] = u[self.i_lo:self.i_lo + i].to(dt)
                self.w2.data[le * h:(le + 1) * h] = d[:, self.i_lo:self.i_lo + i].to(dt)
        if found and self.nvfp4:
            self._refresh_alpha()
        return found

    def _refresh_alpha(self):
        i, h = self.inter, self.cfg.hidden_size
        a13 = self.w13_scale_2.repeat_interleave(i, dim=1).reshape(-1) * self.input_scale
        self.w13_alpha.copy_(self._interleave(a13) if self._w13_interleaved else a13)
        self.w2_alpha.copy_(self.w2_scale_2.repeat_interleave(h) * self.down_input_scale)

    @torch.no_grad()
    def random_init(self, gen: torch.Generator, std: float = 0.02) -> None:
        i, h = self.inter, self.cfg.hidden_size
        dev = self.gate.weight.device

        def draw(shape):
            seed = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=gen))
            g = torch.Generator(device=dev).manual_seed(seed)
            return torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * std

        self.gate.weight.data.copy_(draw(tuple(self.gate.weight.shape)).to(self.gate.weight.dtype))
        for le in range(self.e_local):
            w13, w2 = draw((2 * i, h)), draw((h, i))
            if self.nvfp4:
                for half in range(2):
                    p, sf, gs = ref.nvfp4_quantize(w13[half * i:(half + 1) * i])
                    r0 = le * 2 * i + half * i
                    self.w13[r0:r0 + i] = p
                    self.w13_scale.view(torch.uint8)[r0:r0 + i] = sf.view(torch.uint8)
                    self.w13_scale_2[le, half] = gs
                p, sf, gs = ref.nvfp4_quantize(w2)
                self.w2[le * h:(le + 1) * h] = p
                self.w2_scale.view(torch.uint8)[le * h:(le + 1) * h] = sf.view(torch.uint8)
                self.w2_scale_2[le] = gs
            else:
                self.w13.data[le * 2 * i:(le + 1) * 2 * i] = w13.to(self.w13.dtype)
                self.w2.data[le * h:(le + 1) * h] = w2.to(self.w2.dtype)
        if self.nvfp4:
            self._refresh_alpha()

    _w13_interleaved = False      # gate / up rows of every expert alternate in blocks of 64 (set by finalize on the GPU)

    def _interleave(self, t: torch.Tensor, inverse: bool = False) -> torch.Tensor:
        """[E * 2I, ...] with each expert's rows as [gate I | up I]  <->  blocks of 64 gate rows, 64 up rows, ..."""
        e, i = self.e_local, self.inter
        rest = t.shape[1:]
        if inverse:
            return t.reshape(e, i // 64, 2, 64, *rest).transpose(1, 2).reshape(e * 2 * i, *rest)
        return t.reshape(e, 2, i // 64, 64, *rest).transpose(1, 2).reshape(e * 2 * i, *rest)

    def finalize(self):
        if self.nvfp4 and self.w13.is_cuda:
            cu = ops.cuda_ops()
            if (not self._w13_interleaved and self.inter % 64 == 0
                    and os.environ.get("TELB_MOE_SWIGLU_FUSION", "0") == "1"):
                # Opt-in: the expert gate/up GEMM applies SwiGLU + quantisation in its epilogue (a 128-wide output tile then
                # holds 64 gate features and the matching 64 up features).  Off by default because it measured slower on a
                # B200: expert GEMMs have short K loops (hidden 2048 = 8 K steps), so the epilogue sits on the critical path
                # and one row per lane leaves most lanes idle on the sparsely filled tiles of a decode step (FC1 58.6 -> 89.1 us
                # at 32 tokens, 311 -> 398 us at 8192 tokens, Qwen3-30B-A3B shape); the separate element-wise kernel wins.
                self.w13.copy_(self._interleave(self.w13))
                self.w13_scale.view(torch.uint8).copy_(self._interleave(self.w13_scale.view(torch.uint8)))
                self.w13_alpha.copy_(self._interleave(self.w13_alpha))
                self._w13_interleaved = True
            self._w13_sf = cu.nvfp4_swizzle_scales(self.w13_scale)
            self._w2_sf = cu.nvfp4_swizzle_scales(self.w2_scale)

    # ---- forward ---------------------------------------------------------------------------------
    def _dense_weights(self):
        i, h, e = self.inter, self.cfg.hidden_size, self.e_local
        if self.nvfp4:
            ones = torch.ones((), device=self.w13.device)
            w13q, w13s = self.w13, self.w13_scale
            if self._w13_interleaved:
                w13q = self._interleave(w13q, inverse=True)
                w13s = self._interleave(w13s.view(torch.uint8), inverse=True).view(torch.float8_e4m3fn)
            w13 = ref.nvfp4_dequantize(w13q, w13s, ones) * self.w13_scale_2.repeat_interleave(i, dim=1).reshape(-1, 1)
            w2 = ref.nvfp4_dequantize(self.w2, self.w2_scale, ones) * self.w2_scale_2.repeat_interleave(h).reshape(-1, 1)
            return w13.view(e, 2 * i, h), w2.view(e, h, i)
        return self.w13.view(e, 2 * i, h), self.w2.view(e, h, i)

    ep_comm = None      # a communicator with `moe_all_to_all` (set by the model when experts are sharded over ranks)

    def _shared(self, x: torch.Tensor) -> torch.Tensor:
        """sigmoid(gate · x) ⊙ shared_expert(x) for every row (this rank's partial sum under tensor parallelism)."""
        w = self.shared_expert_gate.weight
        if x.is_cuda:
            if self._gate8 is None or self._gate8.device != x.device:
                self._gate8 = torch.cat([w, torch.zeros(7, w.shape[1], dtype=w.dtype, device=w.device)]).contiguous()
            g = ops.linear(x, self._gate8)[:, :1]
        else:
            g = (x.float() @ w.float().t()).to(x.dtype)
        return (torch.sigmoid(g.float()) * self.shared_expert(x).float()).to(x.dtype)

    def forward(self, x):
        if self.shared_expert is None:
            return self._forward_routed(x)
        if self.ep_comm is not None and self.ep_size > 1 and self.ep_comm.use_ep_all_to_all(x.shape[0]):
            raise NotImplementedError("shared experts are not combined with the token-sharded expert all-to-all")
        return self._forward_routed(x) + self._shared(x)

    def expert_fc1(self, a, ws):
        """NVFP4 rows of the padded expert layout → quantised SwiGLU activations for the second expert GEMM."""
        cu = ops.cuda_ops()
        if self._w13_interleaved:
            return cu.gemm_grouped_swiglu(a, self.w13, ws, self.e_local, self.w13_alpha, self._w13_sf, self.down_input_scale)
        h1 = cu.gemm_grouped(a, self.w13, ws, self.e_local, alpha=self.w13_alpha, w_sf=self._w13_sf)
        return cu.swiglu_quant(h1, self.down_input_scale, moe_ws=ws)

    def _forward_routed(self, x):
        if isinstance(x, torch.Tensor) and not x.is_cuda:
            return self._forward_reference(x)
        if self.ep_comm is not None and self.ep_size > 1 and self.ep_comm.use_ep_all_to_all(x.shape[0]):
            return self.ep_comm.moe_all_to_all(self, x)       # prefill: token-sharded all-to-all over peer memory
        cu = ops.cuda_ops()
        xa = x            # the router always sees 16-bit activations
        logits = self.gate(xa)
        w, idx = cu.moe_route_softmax_topk(logits, self.top_k, self.cfg.norm_topk_prob)
        ws = cu.moe_align(idx, self.num_experts, self.e_lo, self.e_hi)
        if self.nvfp4:
            if self._w13_sf is None:
                self.finalize()
            a = cu.moe_gather(xa, ws, self.top_k, self.input_scale)
            a2 = self.expert_fc1(a, ws)
            y = cu.gemm_grouped(a2, self.w2, ws, self.e_local, alpha=self.w2_alpha, w_sf=self._w2_sf)
        else:
            a = cu.moe_gather(xa, ws, self.top_k, None)
            h1 = cu.gemm_grouped(a, self.w13, ws, self.e_local)
            y = cu.gemm_grouped(cu.swiglu(h1), self.w2, ws, self.e_local)
        return cu.moe_combine(y, ws, w)

    def _forward_reference(self, x):
        logits = self.gate(x)
        w, idx = ref.moe_route_softmax_topk(logits, self.top_k, self.cfg.norm_topk_prob)
        w13, w2 = self._dense_weights()
        local = idx - self.e_lo
        mask = (idx >= self.e_lo) & (idx < self.e_hi)
        xin = x
        if self.nvfp4:
            xin = ref.nvfp4_act_qdq(x, self.input_scale)
        out = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32, device=x.device)
        for e in range(self.e_local):
            rows, slot = ((local == e) & mask).nonzero(as_tuple=True)
            if rows.numel() == 0:
                continue
            hmid = xin[rows].float() @ w13[e].float().t()
            g, u = hmid.to(x.dtype).float().chunk(2, dim=-1)
            act = (torch.nn.functional.silu(g) * u).to(x.dtype)
            if self.nvfp4:
                act = ref.nvfp4_act_qdq(act, self.down_input_scale)
            ye = (act.float() @ w2[e].float().t()).to(x.dtype).float()
            out.index_add_(0, rows, ye * w[rows, slot].float()[:, None])
        return out.to(x.dtype)


class MoEDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int):
        super().__init__()
        p = f"model.layers.{layer_idx}"
        self.self_attn = Attention(cfg, layer_idx, f"{p}.self_attn")
        self.mlp = MoEBlock(cfg, f"{p}.mlp")
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)

    def forward(self, h, residual, meta, kv_layer, cos_sin, comm):
        qs_attn = self.self_attn.qkv_proj.fused_input_scale()
        if residual is None:
            residual = h
            x = ops.rmsnorm_maybe_quant(h, self.input_layernorm.weight, self.input_layernorm.eps, qs_attn)
        else:
            x, residual = comm.add_rmsnorm(h, residual, self.input_layernorm.weight, self.input_layernorm.eps, qs_attn)
        a = self.self_attn(x, meta, kv_layer, cos_sin)
        x, residual = comm.add_rmsnorm(a, residual, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps)
        return self.mlp(x), residual


class MoETransformer(Transformer):
    def __init__(self, cfg: ModelConfig):
        nn.Module.__init__(self)
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=cfg.compute_dtype)
        self.embed_tokens.weight.requires_grad_(False)
        self.layers = nn.ModuleList([MoEDecoderLayer(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)


@register_model("qwen3_moe", "qwen2_moe", "mixtral")
class MoECausalLM(CausalLM):
    transformer_cls = MoETransformer

    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__(cfg, comm)
        if cfg.mapping.ep_size > 1 and hasattr(self.comm, "moe_all_to_all"):
            # Prefill-size steps keep the residual stream token-sharded: the attention output leaves through the
            # reduce-scatter epilogue and the experts exchange token rows all-to-all (see FusedComm).
            for layer in self.model.layers:
                layer.self_attn.o_proj.rs_comm = self.comm
                layer.mlp.ep_comm = self.comm
