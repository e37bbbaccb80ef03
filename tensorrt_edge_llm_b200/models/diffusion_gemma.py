"""Block-diffusion language model on the Gemma text stack.

The backbone is the Gemma decoder of ``models/gemma.py``.  Generation does not append one token per pass: a *canvas* of
``canvas_length`` token ids is denoised as a whole, every canvas row attending to the committed history and to every other
canvas row.  Between passes the model is *self-conditioned*: the previous pass's output distribution, taken at the pass's
temperature, is turned into one expected embedding per row (``softmax(logits / T) @ E``), and a small gated MLP folds that
soft embedding into the embedding of the row's current token::

    inputs = post_norm(E[canvas] + down(gelu_tanh(gate(pre_norm(soft))) * up(pre_norm(soft))))

The decoder that drives the passes is ``runtime/block_diffusion.py``.

Parity: ``tensorrt_edgellm/models/diffusion_gemma/modeling_diffusion_gemma.py`` (``DiffusionGemmaSelfConditioning`` :693,
``_unified_conditioned_inputs`` :312, ``_next_self_conditioning_embeds`` :326, the checkpoint key map :48).  Checkpoints keep
the text stack under ``model.decoder.*``; the encoder tower (vision weights, per-phase layer scalars) is not loaded."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..config import DiffusionConfig, ModelConfig
from ..model import register_model
from .default import RMSNorm
from .gemma import GemmaCausalLM
from .linear import TPMode, make_linear


class SelfConditioning(nn.Module):
    """Gated MLP that mixes the previous pass's expected embedding into the token embedding."""

    def __init__(self, cfg: ModelConfig, size: int):
        super().__init__()
        h = cfg.hidden_size
        self.pre_norm = RMSNorm(h, cfg.rms_norm_eps, cfg.compute_dtype)
        self.gate_up_proj = make_linear(cfg, "self_conditioning.gate_up_proj", h, [size, size], TPMode.COL, sources=["gate_proj", "up_proj"])
        self.down_proj = make_linear(cfg, "self_conditioning.down_proj", size, [h], TPMode.ROW)
        # checkpoints carry no post-norm weight: the unit weight makes it a weightless RMS norm
        self.post_norm = RMSNorm(h, cfg.rms_norm_eps, cfg.compute_dtype)

    def forward(self, token_embeds: torch.Tensor, soft_embeds: torch.Tensor, comm) -> torch.Tensor:
        x = ops.rmsnorm(soft_embeds, self.pre_norm.weight, self.pre_norm.eps)
        sc = comm.all_reduce(self.down_proj(ops.geglu(self.gate_up_proj(x), True)))
        return ops.rmsnorm((token_embeds.float() + sc.float()).to(token_embeds.dtype), self.post_norm.weight, self.post_norm.eps)


@register_model("diffusion_gemma")
class DiffusionGemmaLM(GemmaCausalLM):
    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__(cfg, comm)
        if cfg.diffusion is None:
            cfg.diffusion = DiffusionConfig()
        self.diffusion: DiffusionConfig = cfg.diffusion
        size = self.diffusion.self_conditioning_size or cfg.intermediate_size
        self.self_conditioning = SelfConditioning(cfg, size) if self.diffusion.self_conditioning_enabled else None

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        if key.startswith("model.decoder.self_conditioning."):
            return "self_conditioning." + key[len("model.decoder.self_conditioning."):]
        if key.startswith("model.decoder."):
            return "model." + key[len("model.decoder."):]
        if key.startswith("model.encoder."):
            return None
        return key

    # ---- the two halves of self-conditioning ------------------------------------------------
    def scaled_embedding(self) -> torch.Tensor:
        """Embedding table with Gemma's ``sqrt(hidden)`` multiplier applied (a loaded checkpoint has it folded in)."""
        w = self.model.embed_tokens.weight
        s = self.model.embed_scale
        return w if s == 1.0 else (w * torch.tensor(s, dtype=w.dtype)).to(w.dtype)

    def canvas_inputs(self, canvas_ids: torch.Tensor, soft_embeds: Optional[torch.Tensor]) -> torch.Tensor:
        """Input rows ``[T, H]`` of a denoise pass: token embeddings, conditioned on ``soft_embeds`` (``None`` = zeros)."""
        tok = ops.embedding(canvas_ids.to(torch.int32), self.model.embed_tokens.weight)
        if self.model.embed_scale != 1.0:
            tok = (tok * torch.tensor(self.model.embed_scale, dtype=tok.dtype)).to(tok.dtype)
        if self.self_conditioning is None:
            return tok
        if soft_embeds is None:
            soft_embeds = torch.zeros_like(tok)
        return self.self_conditioning(tok, soft_embeds.to(tok.dtype), self.comm)

    def soft_embeddings(self, logits: torch.Tensor, temperature: float) -> torch.Tensor:
        """Expected embedding of every row under ``softmax(logits / temperature)``; feeds the next pass."""
        probs = torch.softmax(logits.float() / max(float(temperature), 1e-6), dim=-1)
        table = self.scaled_embedding()
        cols = probs.shape[-1]
        if cols != table.shape[0]:                       # a reduced LM head covers a subset of the table's rows
            raise ValueError("self-conditioning needs logits over the whole vocabulary")
        return (probs.to(table.dtype) @ table).to(table.dtype)

    @torch.no_grad()
    def finalize_checkpoint(self):
        super().finalize_checkpoint()
        if self.self_conditioning is not None:
            # the base class added one to every norm weight (stored-minus-one convention); the post-norm has no stored
            # weight, so it went from one to two: put the unit weight back
            self.self_conditioning.post_norm.weight.fill_(1.0)
