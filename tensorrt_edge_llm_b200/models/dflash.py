"""DFlash block draft: proposes a whole block of tokens in one forward pass.

The draft is a small decoder whose attention *context* is not its own past hidden states but the target model's: the
hidden states of a few tapped target layers are concatenated, projected (``fc``) and normalised once per accepted token,
and every draft layer turns those rows into keys and values with its own ``k_proj`` / ``v_proj`` (k-norm and RoPE at the
token's position) and keeps them in a paged draft cache.  A proposal is the block ``[y0, mask, …, mask]`` — the last
accepted token followed by mask tokens — run through the layers with attention over the cached context plus the block
itself (every block row sees every other one); row ``i`` of the output gives the token at offset ``i`` after ``y0``.

Here one draft forward is two ragged steps over the same weights:

* ``write_context(features, meta)`` — per layer, QKV GEMM over the new context rows and the RoPE + KV-write kernel; no
  attention (the rows' outputs are never used),
* ``propose(embeds, meta)`` — an ordinary ragged step of ``block`` rows per sequence with a full tree mask.

Parity: ``tensorrt_edgellm/models/dflash/modeling_dflash_draft.py`` (``DFlashCachedAttention`` :118, layer :390, model :552;
``dflash_target_kv_cache_update`` is the context write, the tree-attention plugin call the proposal step) and
``tensorrt_edgellm/config.py:848-895`` for the configuration fields."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from ..parallel.comm import LocalComm
from .default import MLP, Attention, RMSNorm
from .linear import TPMode, make_linear


class DFlashLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int):
        super().__init__()
        p = f"layers.{idx}"
        self.self_attn = Attention(cfg, idx, f"{p}.self_attn")
        self.mlp = MLP(cfg, f"{p}.mlp")
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)

    def write_context(self, h_ctx, meta, kv_layer, cos_sin):
        """Keys / values of the projected target rows (not normalised by this layer) into the draft cache."""
        a = self.self_attn
        qkv = a.qkv_proj(h_ctx)
        ops.rope_kv_write(qkv, kv_layer, meta, cos_sin, a.num_q_heads, a.num_kv_heads, a.head_dim,
                          None if a.q_norm is None else a.q_norm.weight, None if a.k_norm is None else a.k_norm.weight, a.eps)

    def forward(self, h, meta, kv_layer, cos_sin, comm):
        x = ops.rmsnorm(h, self.input_layernorm.weight, self.input_layernorm.eps)
        h = h + comm.all_reduce(self.self_attn(x, meta, kv_layer, cos_sin))
        x = ops.rmsnorm(h, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps)
        return h + comm.all_reduce(self.mlp(x))


@register_model("dflash", "dflash_draft")
class DFlashDraft(nn.Module):
    packed_modules = {"qkv_proj": ["q_proj", "k_proj", "v_proj"], "gate_up_proj": ["gate_proj", "up_proj"]}

    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__()
        self.cfg = cfg
        self.comm = comm or LocalComm()
        taps = len(cfg.dflash_target_layer_ids) or 3
        ht = cfg.eagle3_target_hidden_size or cfg.hidden_size
        self.fc = make_linear(cfg, "fc", taps * ht, [cfg.hidden_size], TPMode.REPLICATED, quantizable=False)
        self.hidden_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)
        self.layers = nn.ModuleList([DFlashLayer(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.compute_dtype)
        self.lm_head = make_linear(cfg, "lm_head", cfg.hidden_size, [cfg.vocab_size], TPMode.REPLICATED, quantizable=False)
        self.embed_tokens: Optional[nn.Module] = None          # the target's table (share_with)
        self._cos_sin: Optional[torch.Tensor] = None

    def share_with(self, target) -> None:
        """Use the target's token table (the block is embedded with it) and, when the draft checkpoint brought no head of its
        own, the target's LM head."""
        self.embed_tokens = target.model.embed_tokens
        if float(self.lm_head.weight.abs().sum()) == 0.0 and tuple(self.lm_head.weight.shape) == tuple(target.lm_head.weight.shape):
            self.lm_head = target.lm_head

    share_lm_head = share_with

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        return key[len("model."):] if key.startswith("model.") else key

    def cos_sin(self, device) -> torch.Tensor:
        if self._cos_sin is None or self._cos_sin.device != torch.device(device):
            self._cos_sin = ops.rope_cos_sin(self.cfg.max_position_embeddings, self.cfg.rotary_dim, self.cfg.rope_theta,
                                                 self.cfg.rope_scaling, device=device)
        return self._cos_sin

    def project(self, target_hidden: torch.Tensor) -> torch.Tensor:
        """Tapped target hidden states ``[T, taps · H_target]`` → context rows ``[T, H]``.  The projection accumulates in
        fp32: target hidden states of large models exceed the fp16 range before the norm brings them back."""
        w = self.fc.weight
        acc = target_hidden.float() @ w.float().t()
        acc = acc * torch.rsqrt(acc.pow(2).mean(-1, keepdim=True) + self.hidden_norm.eps) * self.hidden_norm.weight.float()
        return acc.to(self.cfg.compute_dtype)

    @torch.no_grad()
    def write_context(self, target_hidden: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor) -> None:
        h = self.project(target_hidden)
        cs = self.cos_sin(h.device)
        for i, layer in enumerate(self.layers):
            layer.write_context(h, meta, kv_pool[i], cs)

    @torch.no_grad()
    def block_hidden(self, embeds: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor) -> torch.Tensor:
        """Normalised hidden state ``[T, H]`` of every proposal row, aligned so that row ``i`` of a block describes the token
        at offset ``i`` after the block's first token (with shifted labels the row is the hidden state of row ``i - 1``)."""
        h = embeds.to(self.cfg.compute_dtype)
        cs = self.cos_sin(h.device)
        for i, layer in enumerate(self.layers):
            h = layer(h, meta, kv_pool[i], cs, self.comm)
        if self.cfg.dflash_shift_label:
            first = meta.q_start[:-1].long()
            shifted = torch.roll(h, 1, dims=0)
            shifted[first] = h[first]
            h = shifted
        return ops.rmsnorm(h, self.norm.weight, self.norm.eps)

    def head(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.lm_head(x).float()
        cap = self.cfg.final_logit_softcapping
        return torch.tanh(logits / cap) * cap if cap else logits

    @torch.no_grad()
    def propose(self, embeds: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor) -> torch.Tensor:
        """Logits ``[T, V]`` (fp32) of the proposal rows; ``meta.tree_mask`` lets every row of a block see the whole block."""
        return self.head(self.block_hidden(embeds, meta, kv_pool))


@register_model("domino", "domino_draft")
class DominoDraft(DFlashDraft):
    """DFlash backbone plus the Domino correction head.

    The block's proposals are not taken independently.  A candidate pool — the ``P`` tokens with the largest logit at any
    proposal position — is scored per position; the first proposal is the pool's best token at position 1, and every later
    position ``i`` is corrected by what was chosen before it: a bias-free GRU reads the chosen tokens, and

        c      = SiLU(z_projection(hidden_i) + proj_state · h_gru)
        score  = base_logits_i[pool] + codebook[pool] · c
        token  = pool[argmax score]

    Parity: ``tensorrt_edgellm/models/domino/modeling_domino_draft.py`` (pool outputs :107-140) and
    ``cpp/runtime/decoding/dominoDecoder.cpp:160`` / ``cpp/kernels/speculative/dominoRolloutKernels.h`` (rollout: first
    proposal, GRU seeded with the last accepted token and the first proposal, one correction + GRU update per position).
    The pool holds a few thousand candidates, so the rollout is torch ops over ``[batch, P]`` tensors."""

    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__(cfg, comm)
        dt, r, g = cfg.compute_dtype, cfg.domino_proj_dim, cfg.domino_gru_hidden_dim
        mk = lambda *shape: nn.Parameter(torch.zeros(*shape, dtype=dt), requires_grad=False)
        self.z_projection = mk(r, cfg.hidden_size)            # checkpoint: domino_pool.z_projection.weight
        self.codebook = mk(cfg.vocab_size, r)                 # domino_pool.codebook
        self.gru_input_table = mk(cfg.vocab_size, 3 * g)      # W_ih · embedding(token), gate order r, z, n
        self.gru_weight_hh = mk(3 * g, g)
        self.proj_state_weight = mk(r, g)

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        key = DFlashDraft.checkpoint_key_remap(key)
        return {"domino_pool.z_projection.weight": "z_projection", "domino_pool.codebook": "codebook"}.get(key, key)

    def gru(self, tokens: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        g = h.shape[-1]
        x = self.gru_input_table[tokens.long()].float()
        hh = h @ self.gru_weight_hh.float().t()
        r = torch.sigmoid(x[:, :g] + hh[:, :g])
        z = torch.sigmoid(x[:, g:2 * g] + hh[:, g:2 * g])
        n = torch.tanh(x[:, 2 * g:] + r * hh[:, 2 * g:])
        return (1 - z) * n + z * h

    @torch.no_grad()
    def propose_tokens(self, embeds: torch.Tensor, meta: StepMeta, kv_pool: torch.Tensor, last_accepted: torch.Tensor, block: int
                       ) -> torch.Tensor:
        """Draft tokens ``[N, block - 1]`` for blocks whose first token is ``last_accepted [N]``."""
        x = self.block_hidden(embeds, meta, kv_pool)
        n = x.shape[0] // block
        hid = x.reshape(n, block, -1)[:, 1:, :]                                   # proposal positions 1 .. block-1
        logits = self.head(hid.reshape(n * (block - 1), -1)).reshape(n, block - 1, -1)
        pool = torch.topk(logits.amax(dim=1), min(self.cfg.domino_pool_size, logits.shape[-1]), dim=-1).indices      # [N, P]
        base = torch.gather(logits, 2, pool[:, None, :].expand(-1, block - 1, -1))                                   # [N, B-1, P]
        code = self.codebook[pool].float()                                                                           # [N, P, R]
        zproj = hid[:, 1:, :].float() @ self.z_projection.float().t()                                                # [N, B-2, R]
        out = torch.empty(n, block - 1, dtype=torch.int64, device=x.device)
        pick = lambda score: torch.gather(pool, 1, score.argmax(-1, keepdim=True))[:, 0]      # ties → the first (best-ranked) slot
        out[:, 0] = pick(base[:, 0])
        h = torch.zeros(n, self.cfg.domino_gru_hidden_dim, device=x.device)
        h = self.gru(last_accepted, h)
        h = self.gru(out[:, 0], h)
        for step in range(block - 2):
            c = torch.nn.functional.silu(zproj[:, step] + h @ self.proj_state_weight.float().t())
            out[:, step + 1] = pick(base[:, step + 1] + torch.einsum("npr,nr->np", code, c))
            if step + 1 < block - 2:
                h = self.gru(out[:, step + 1], h)
        return out
