"""Embedding tables stored in FP8 or NVFP4 and expanded on lookup.

The reference keeps its embedding table outside the engine as ``EmbeddingData`` in FP16, FP8 or NVFP4
(``cpp/runtime/llmRuntimeUtils.h:522-548``) and dequantises the gathered rows (``cpp/kernels/embeddingKernels``).  Here
:class:`QuantizedEmbedding` replaces a model's ``embed_tokens``: rows are gathered in their stored form — one byte (FP8,
with an fp32 scale per row) or half a byte plus one E4M3 scale per 16 values (NVFP4) per element — and expanded to the
compute type, so a 151936 × 4096 table takes 0.62 GB or 0.35 GB instead of 1.24 GB.  Only the step's rows are expanded."""
from __future__ import annotations

import torch
from torch import nn

from ..ops import reference as ref


class QuantizedTable:
    """What ``ops.embedding(ids, table)`` receives in place of a dense weight."""

    def __init__(self, owner: "QuantizedEmbedding"):
        self.owner = owner

    @property
    def shape(self):
        return (self.owner.num_embeddings, self.owner.embedding_dim)

    @property
    def is_cuda(self) -> bool:
        return self.owner.data.is_cuda

    @property
    def device(self):
        return self.owner.data.device

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        return self.owner(ids)


class QuantizedEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, fmt: str, dtype=torch.bfloat16):
        super().__init__()
        if fmt not in ("fp8", "nvfp4"):
            raise ValueError("embedding format must be fp8 or nvfp4")
        if fmt == "nvfp4" and embedding_dim % 16:
            raise ValueError("NVFP4 rows need a multiple of 16 features")
        self.num_embeddings, self.embedding_dim, self.fmt, self.out_dtype = num_embeddings, embedding_dim, fmt, dtype
        if fmt == "fp8":
            self.register_buffer("data", torch.zeros(num_embeddings, embedding_dim, dtype=torch.float8_e4m3fn))
            self.register_buffer("scale", torch.ones(num_embeddings, dtype=torch.float32))
        else:
            self.register_buffer("data", torch.zeros(num_embeddings, embedding_dim // 2, dtype=torch.uint8))
            self.register_buffer("scale", torch.zeros(num_embeddings, embedding_dim // 16, dtype=torch.float8_e4m3fn))
            self.register_buffer("global_scale", torch.ones((), dtype=torch.float32))

    @classmethod
    @torch.no_grad()
    def from_dense(cls, weight: torch.Tensor, fmt: str) -> "QuantizedEmbedding":
        m = cls(weight.shape[0], weight.shape[1], fmt, weight.dtype).to(weight.device)
        w = weight.float()
        if fmt == "fp8":
            s = (w.abs().amax(1) / 448.0).clamp(min=1e-12)
            m.data.copy_((w / s[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn))
            m.scale.copy_(s)
        else:
            for r0 in range(0, w.shape[0], 16384):             # chunks keep the fp32 staging small for large vocabularies
                if r0 == 0:
                    gs = (w.abs().amax() / (6.0 * 448.0)).clamp(min=1e-12)
                    m.global_scale.copy_(gs)
                p, sf, _ = ref.nvfp4_quantize(w[r0:r0 + 16384], m.global_scale)
                m.data[r0:r0 + 16384].copy_(p)
                m.scale[r0:r0 + 16384].copy_(sf.view(torch.float8_e4m3fn))
        return m

    @property
    def weight(self) -> QuantizedTable:
        return QuantizedTable(self)

    def table_bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.buffers())

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if self.data.is_cuda and self.out_dtype in (torch.float16, torch.bfloat16) and self.embedding_dim % 16 == 0:
            from ..ops import cuda as cu           # one kernel: gather and expand (csrc/kernels/elementwise.cu)
            out = cu.embedding_quant(ids.reshape(-1), self.data, self.scale, getattr(self, "global_scale", None), self.fmt, self.out_dtype)
            return out.reshape(*ids.shape, self.embedding_dim)
        idx = ids.long()
        if self.fmt == "fp8":
            return (self.data[idx].float() * self.scale[idx][..., None]).to(self.out_dtype)
        return ref.nvfp4_dequantize(self.data[idx], self.scale[idx], self.global_scale).to(self.out_dtype)


@torch.no_grad()
def quantize_embedding(model, fmt: str):
    """Swap ``model.model.embed_tokens`` for its FP8 / NVFP4 form (the LM head keeps its own weights)."""
    t = model.model
    emb = t.embed_tokens
    if isinstance(emb, QuantizedEmbedding):
        return emb
    t.embed_tokens = QuantizedEmbedding.from_dense(emb.weight.data, fmt)
    return t.embed_tokens
