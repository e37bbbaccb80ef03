"""Hybrid decoder: Mamba2-SSD, gated-DeltaNet and GQA-attention mixers with dense MLPs.

Parity: ``tensorrt_edgellm/models/nemotron_h/modeling_nemotron_h.py`` — ``MambaMixer`` wiring
(:239-446: ``in_proj → [z | conv-in (x‖B‖C) | dt]``, conv1d + SiLU, ``A = −exp(A_log)``, selective
state update, gated group-RMSNorm, ``out_proj``; dt clamp), relu² MLP (:555-573) — and the gated
DeltaNet mixer of ``tensorrt_edgellm/models/qwen3_5/modeling_qwen3_5_text.py:162-379`` (``in_proj_qkv
‖ z ‖ b ‖ a``, conv1d + SiLU, delta rule, per-head RMSNorm · silu(z), ``out_proj``).

A layer is ``x += mixer(norm(x))`` followed by ``x += mlp(norm(x))``; either half may be absent
(``layer_types[i] == "none"`` / ``mlp_types[i] == "none"``), which covers both the Nemotron-H
block pattern (one mixer *or* one MLP per block) and transformer-style hybrid stacks.  Recurrent
state (conv history, SSM state, delta-rule state) lives in per-layer pools indexed by the step's
``slot_ids``; tensor parallelism shards heads (column-parallel in, row-parallel out).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..config import LAYER_ATTENTION, LAYER_GDN, LAYER_MAMBA, LAYER_MLP, LAYER_MOE, ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from .default import MLP, Attention, CausalLM, RMSNorm
from .linear import TPMode, make_linear


class RecurrentState:
    """Per-layer state pools of the recurrent mixers (rows = seats)."""

    def __init__(self, cfg: ModelConfig, seats: int, device, dtype):
        tp = cfg.tp_size
        self.conv, self.ssm, self.gdn = {}, {}, {}
        for i, t in enumerate(cfg.layer_types):
            if t == LAYER_MAMBA:
                m = cfg.mamba
                conv_dim = (m.intermediate_size + 2 * m.n_groups * m.d_state) // tp
                self.conv[i] = torch.zeros(seats, conv_dim, m.conv_kernel - 1, dtype=dtype, device=device)
                self.ssm[i] = torch.zeros(seats, m.num_heads // tp, m.head_dim, m.d_state, dtype=torch.float32, device=device)
            elif t == LAYER_GDN:
                g = cfg.gdn
                self.conv[i] = torch.zeros(seats, g.conv_dim // tp, g.conv_kernel - 1, dtype=dtype, device=device)
                self.gdn[i] = torch.zeros(seats, g.num_v_heads // tp, g.head_k_dim, g.head_v_dim, dtype=torch.float32, device=device)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for d in (self.conv, self.ssm, self.gdn) for t in d.values())

    def pools(self):
        for d in (self.conv, self.ssm, self.gdn):
            yield from d.values()

    # ---- replay data -------------------------------------------------------------------------------------------------
    # A speculative verification step advances every state over the whole draft chain.  While ``record`` is a dict the mixers
    # also keep the inputs of their recurrent kernels for that step (a few KB per token and layer); when only a prefix of
    # the chain is accepted, ``HybridCausalLM.replay_recurrent`` restores the saved rows and runs *only the recurrent kernels*
    # over the accepted tokens again from those inputs: no projections, no attention, no MLP.
    record = None

    def begin_record(self) -> None:
        self.record = {}

    def end_record(self):
        rec, self.record = self.record, None
        return rec

    def snapshot(self, seats) -> list:
        """Copies of the state rows of ``seats`` (the commit policy of speculative verification restores them when a
        draft chain is only partly accepted; ``cpp/runtime/commitPolicy/`` in the reference)."""
        idx = torch.as_tensor(list(seats), dtype=torch.long, device=next(self.pools()).device)
        return [t.index_select(0, idx) for t in self.pools()]

    def restore(self, seats, snap: list, which=None) -> None:
        """Write back the rows of ``snap`` for ``seats`` (all of them, or the positions listed in ``which``)."""
        sel = list(range(len(seats))) if which is None else list(which)
        if not sel:
            return
        dev = next(self.pools()).device
        dst = torch.as_tensor([seats[j] for j in sel], dtype=torch.long, device=dev)
        src = torch.as_tensor(sel, dtype=torch.long, device=dev)
        for t, saved in zip(self.pools(), snap):
            t.index_copy_(0, dst, saved.index_select(0, src))


class MambaMixer(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        m, tp = cfg.mamba, cfg.tp_size
        self.m = m
        self.nheads = m.num_heads // tp
        self.groups = max(m.n_groups // tp, 1)
        if m.num_heads % tp or m.n_groups % tp:
            raise ValueError("Mamba heads and groups must divide over the TP ranks")
        self.d_inner = self.nheads * m.head_dim
        self.bc = self.groups * m.d_state
        di, gn = m.intermediate_size, m.n_groups * m.d_state
        # one checkpoint tensor in_proj.weight = [z | x | B | C | dt]; each segment is sharded on its own
        self.in_proj = make_linear(cfg, f"{prefix}.in_proj", cfg.hidden_size, [di, di, gn, gn, m.num_heads], TPMode.COL)
        self.out_proj = make_linear(cfg, f"{prefix}.out_proj", di, [cfg.hidden_size], TPMode.ROW)
        conv_dim = self.d_inner + 2 * self.bc
        dt = cfg.compute_dtype
        self.conv_weight = nn.Parameter(torch.zeros(conv_dim, m.conv_kernel, dtype=dt), requires_grad=False)
        self.conv_bias = nn.Parameter(torch.zeros(conv_dim, dtype=dt), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.nheads, dtype=torch.float32), requires_grad=False)
        self.D = nn.Parameter(torch.ones(self.nheads, dtype=torch.float32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(self.nheads, dtype=torch.float32), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(self.d_inner, dtype=dt), requires_grad=False)
        self.eps = cfg.rms_norm_eps
        self.prefix, self.cfg = prefix, cfg

    @torch.no_grad()
    def load_checkpoint(self, fetch) -> bool:
        w = fetch(f"{self.prefix}.conv1d.weight")
        if w is None:
            return False
        m, tp, r = self.m, self.cfg.tp_size, self.cfg.tp_rank
        di, gn = m.intermediate_size, m.n_groups * m.d_state

        def seg(t):     # shard [x | B | C] stacked along dim 0
            parts = [t[:di], t[di:di + gn], t[di + gn:di + 2 * gn]]
            return torch.cat([p.chunk(tp, 0)[r] for p in parts], 0)

        self.conv_weight.copy_(seg(w.reshape(w.shape[0], -1)).to(self.conv_weight.dtype))
        b = fetch(f"{self.prefix}.conv1d.bias")
        if b is not None:
            self.conv_bias.copy_(seg(b).to(self.conv_bias.dtype))
        for name, dst in (("A_log", self.A_log), ("D", self.D), ("dt_bias", self.dt_bias)):
            t = fetch(f"{self.prefix}.{name}")
            if t is not None:
                dst.copy_(t.float().chunk(tp, 0)[r])
        nw = fetch(f"{self.prefix}.norm.weight")
        if nw is not None:
            self.norm_weight.copy_(nw.chunk(tp, 0)[r].to(self.norm_weight.dtype))
        return False        # linear layers are still loaded by the generic path

    @torch.no_grad()
    def random_init(self, gen, std=0.02):
        self.conv_weight.copy_((torch.randn(self.conv_weight.shape, generator=gen) * 0.3).to(self.conv_weight.dtype))
        self.A_log.copy_(torch.log(torch.rand(self.nheads, generator=gen) * 3 + 1))
        self.dt_bias.copy_(torch.rand(self.nheads, generator=gen) - 2.0)

    def forward(self, x, meta: StepMeta, state: RecurrentState, layer_idx: int):
        m = self.m
        proj = self.in_proj(x)
        z, xbc, dt = proj.split([self.d_inner, self.d_inner + 2 * self.bc, self.nheads], dim=-1)
        if state.record is not None:
            state.record[layer_idx] = (xbc.contiguous(), dt.contiguous())
        xbc = ops.causal_conv1d(xbc.contiguous(), self.conv_weight, self.conv_bias, state.conv[layer_idx], meta, activation=True)
        xs, B, C = xbc.split([self.d_inner, self.bc, self.bc], dim=-1)
        t = x.shape[0]
        y = ops.ssm_scan(xs.reshape(t, self.nheads, m.head_dim), dt.contiguous(), -torch.exp(self.A_log),
                         B.reshape(t, self.groups, m.d_state), C.reshape(t, self.groups, m.d_state), self.D, self.dt_bias,
                         state.ssm[layer_idx], meta, z=None, dt_softplus=True, dt_limit=m.dt_limit)
        y = ops.gated_group_rmsnorm(y.reshape(t, self.d_inner), z.contiguous(), self.norm_weight, self.groups, self.eps)
        return self.out_proj(y)


    @torch.no_grad()
    def replay(self, saved, rows: torch.Tensor, meta: StepMeta, state: RecurrentState, layer_idx: int) -> None:
        """Advance this layer's convolution and SSM state over the recorded inputs of ``rows`` (the accepted tokens)."""
        m = self.m
        xbc, dt = (t.index_select(0, rows) for t in saved)
        xbc = ops.causal_conv1d(xbc, self.conv_weight, self.conv_bias, state.conv[layer_idx], meta, activation=True)
        xs, B, C = xbc.split([self.d_inner, self.bc, self.bc], dim=-1)
        t = xbc.shape[0]
        ops.ssm_scan(xs.reshape(t, self.nheads, m.head_dim), dt, -torch.exp(self.A_log), B.reshape(t, self.groups, m.d_state),
                     C.reshape(t, self.groups, m.d_state), self.D, self.dt_bias, state.ssm[layer_idx], meta, z=None, dt_softplus=True,
                     dt_limit=m.dt_limit)


class GatedDeltaNetMixer(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        g, tp = cfg.gdn, cfg.tp_size
        self.g = g
        if g.num_k_heads % tp or g.num_v_heads % tp:
            raise ValueError("gated-DeltaNet heads must divide over the TP ranks")
        self.hk, self.hv = g.num_k_heads // tp, g.num_v_heads // tp
        self.key_dim, self.value_dim = self.hk * g.head_k_dim, self.hv * g.head_v_dim
        h = cfg.hidden_size
        self.in_proj_qkv = make_linear(cfg, f"{prefix}.in_proj_qkv", h, [g.key_dim, g.key_dim, g.value_dim], TPMode.COL)
        self.in_proj_z = make_linear(cfg, f"{prefix}.in_proj_z", h, [g.value_dim], TPMode.COL)
        self.in_proj_b = make_linear(cfg, f"{prefix}.in_proj_b", h, [g.num_v_heads], TPMode.COL, quantizable=False)
        self.in_proj_a = make_linear(cfg, f"{prefix}.in_proj_a", h, [g.num_v_heads], TPMode.COL, quantizable=False)
        self.out_proj = make_linear(cfg, f"{prefix}.out_proj", g.value_dim, [h], TPMode.ROW)
        dt = cfg.compute_dtype
        conv_dim = 2 * self.key_dim + self.value_dim
        self.conv_weight = nn.Parameter(torch.zeros(conv_dim, g.conv_kernel, dtype=dt), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.hv, dtype=torch.float32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(self.hv, dtype=torch.float32), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(g.head_v_dim, dtype=dt), requires_grad=False)
        self.eps = cfg.rms_norm_eps
        self.prefix, self.cfg = prefix, cfg

    @torch.no_grad()
    def load_checkpoint(self, fetch) -> bool:
        w = fetch(f"{self.prefix}.conv1d.weight")
        if w is None:
            return False
        g, tp, r = self.g, self.cfg.tp_size, self.cfg.tp_rank
        w = w.reshape(w.shape[0], -1)
        parts = [w[:g.key_dim], w[g.key_dim:2 * g.key_dim], w[2 * g.key_dim:]]
        self.conv_weight.copy_(torch.cat([p.chunk(tp, 0)[r] for p in parts], 0).to(self.conv_weight.dtype))
        for name, dst in (("A_log", self.A_log), ("dt_bias", self.dt_bias)):
            t = fetch(f"{self.prefix}.{name}")
            if t is not None:
                dst.copy_(t.float().chunk(tp, 0)[r])
        nw = fetch(f"{self.prefix}.norm.weight")
        if nw is not None:
            self.norm_weight.copy_(nw.to(self.norm_weight.dtype))
        return False

    @torch.no_grad()
    def random_init(self, gen, std=0.02):
        self.conv_weight.copy_((torch.randn(self.conv_weight.shape, generator=gen) * 0.3).to(self.conv_weight.dtype))
        self.A_log.copy_(torch.log(torch.rand(self.hv, generator=gen) * 3 + 1))
        self.dt_bias.copy_(torch.rand(self.hv, generator=gen) - 2.0)

    def forward(self, x, meta: StepMeta, state: RecurrentState, layer_idx: int):
        g = self.g
        t = x.shape[0]
        qkv = self.in_proj_qkv(x)
        z = self.in_proj_z(x)
        b = self.in_proj_b(x)
        a = self.in_proj_a(x)
        if state.record is not None:
            state.record[layer_idx] = (qkv.contiguous(), a.contiguous(), b.contiguous())
        qkv = ops.causal_conv1d(qkv, self.conv_weight, None, state.conv[layer_idx], meta, activation=True)
        q, k, v = qkv.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        o = ops.gated_delta_rule(q.reshape(t, self.hk, g.head_k_dim), k.reshape(t, self.hk, g.head_k_dim),
                                 v.reshape(t, self.hv, g.head_v_dim), a, b, self.A_log, self.dt_bias, state.gdn[layer_idx], meta)
        # per-head RMSNorm, then the silu(z) gate
        o = ops.rmsnorm(o.reshape(t * self.hv, g.head_v_dim).contiguous(), self.norm_weight, self.eps).reshape(t, self.value_dim)
        zf = z.float()
        o = (o.float() * (zf * torch.sigmoid(zf))).to(x.dtype)
        return self.out_proj(o)


    @torch.no_grad()
    def replay(self, saved, rows: torch.Tensor, meta: StepMeta, state: RecurrentState, layer_idx: int) -> None:
        g = self.g
        qkv, a, b = (t.index_select(0, rows) for t in saved)
        qkv = ops.causal_conv1d(qkv, self.conv_weight, None, state.conv[layer_idx], meta, activation=True)
        q, k, v = qkv.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        t = qkv.shape[0]
        ops.gated_delta_rule(q.reshape(t, self.hk, g.head_k_dim), k.reshape(t, self.hk, g.head_k_dim), v.reshape(t, self.hv, g.head_v_dim),
                             a, b, self.A_log, self.dt_bias, state.gdn[layer_idx], meta)


class HybridLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, i: int):
        super().__init__()
        p = f"model.layers.{i}"
        kind, mlp_kind = cfg.layer_types[i], cfg.mlp_types[i]
        self.kind, self.mlp_kind, self.idx = kind, mlp_kind, i
        dt = cfg.compute_dtype
        if kind == LAYER_ATTENTION:
            self.mixer = Attention(cfg, i, f"{p}.mixer")
        elif kind == LAYER_MAMBA:
            self.mixer = MambaMixer(cfg, f"{p}.mixer")
        elif kind == LAYER_GDN:
            self.mixer = GatedDeltaNetMixer(cfg, f"{p}.mixer")
        else:
            self.mixer = None
        if self.mixer is not None:
            self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dt)
        if mlp_kind == LAYER_MLP:
            self.mlp = MLP(cfg, f"{p}.mlp")
            self.mlp_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dt)
        elif mlp_kind == LAYER_MOE:
            from .qwen3_moe import MoEBlock
            self.mlp = MoEBlock(cfg, f"{p}.mlp")
            self.mlp_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dt)
        else:
            self.mlp = None

    def forward(self, h, residual, meta, cache, cos_sin, comm):
        if self.mixer is not None:
            if residual is None:
                residual = h
                x = self.norm(h)
            else:
                x, residual = comm.add_rmsnorm(h, residual, self.norm.weight, self.norm.eps)
            if self.kind == LAYER_ATTENTION:
                h = self.mixer(x, meta, cache.kv_layer(self.idx), cos_sin)
            else:
                h = self.mixer(x, meta, cache.recurrent, self.idx)
        if self.mlp is not None:
            if residual is None:
                residual = h
                x = self.mlp_norm(h)
            else:
                x, residual = comm.add_rmsnorm(h, residual, self.mlp_norm.weight, self.mlp_norm.eps)
            h = self.mlp(x)
        return h, residual


class HybridTransformer(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=cfg.compute_dtype)
        self.embed_tokens.weight.requires_grad_(False)
        self.layers = nn.ModuleList([HybridLayer(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)

    def forward(self, ids, meta, cache, cos_sin, comm, inputs_embeds=None, capture_layers=()):
        h = ops.embedding(ids, self.embed_tokens.weight) if inputs_embeds is None else inputs_embeds
        residual = None
        taps = []
        for i, layer in enumerate(self.layers):
            h, residual = layer(h, residual, meta, cache, cos_sin, comm)
            if i in capture_layers:
                taps.append((h.float() + residual.float()).to(h.dtype) if comm.world_size == 1 else comm.all_reduce(h).add_(residual))
        x, _ = comm.add_rmsnorm(h, residual, self.norm.weight, self.norm.eps)
        return (x, taps) if capture_layers else x


@register_model("nemotron_h", "nemotron_h_hybrid", "qwen3_next", "qwen3_5")
class HybridCausalLM(CausalLM):
    transformer_cls = HybridTransformer
    needs_cache_set = True      # forward takes the cache manager (KV + recurrent pools), not the bare KV pool

    @torch.no_grad()
    def replay_recurrent(self, record: dict, rows: torch.Tensor, meta: StepMeta, cache) -> int:
        """Advance the recurrent state of every Mamba / DeltaNet layer over the recorded kernel inputs of ``rows`` (row indices into
        the recorded step, grouped by sequence as ``meta`` describes).  The caller has restored the state rows of those sequences
        to what they were before the recorded step.  Returns the number of layers replayed.  This is the commit of a partly
        accepted draft chain on a hybrid target: two small kernels per recurrent layer instead of a second pass through the
        whole model (the reference's per-layer replay data, ``cpp/runtime/commitPolicy``, ``mtpStateScatterKernels``)."""
        n = 0
        for layer in self.model.layers:
            if layer.kind in (LAYER_MAMBA, LAYER_GDN) and layer.idx in record:
                layer.mixer.replay(record[layer.idx], rows, meta, cache.recurrent, layer.idx)
                n += 1
        return n
